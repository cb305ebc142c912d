"""Per-kernel timeline of one decode step.

    python hashattention-1.0_b200/diagnostics/timeline.py [config1|config3] [layer instances] [batch]

Builds a copy of the library with -DHA_TIMELINE next to this file (libhashattn_timeline.so), in which
every CTA stamps %globaltimer at entry, after griddepcontrol.wait and at exit, replays single decode
steps and prints min / max per kernel in microseconds from the first CTA of the encoder kernel."""
import ctypes, os, sys, json
import numpy as np
import torch
import subprocess
HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
sys.path.insert(0, ROOT)
import __graft_entry__ as entry
ha = entry.load_package()
TL_LIB = os.path.join(HERE, "libhashattn_timeline.so")
subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
                "-Xcompiler", "-fPIC", "-DHA_TIMELINE", "-o", TL_LIB, os.path.join(PKG, "csrc", "hashattn_abi.cu")],
               check=True)
ha._lib.LIB_PATH = TL_LIB
lib = ha._lib.load()
lib.ha_debug_set_timeline.restype = ctypes.c_int
lib.ha_debug_set_timeline.argtypes = [ctypes.c_void_p]
from hashattention_b200 import synthetic
import bench

workload = sys.argv[1] if len(sys.argv) > 1 else "config1"
L = int(sys.argv[2]) if len(sys.argv) > 2 else 8
w = bench.WORKLOADS[workload]
lens = bench.workload_lens(workload)
if len(sys.argv) > 3:
    lens = lens[:int(sys.argv[3])]
B = len(lens)
dev = torch.device("cuda:0")
budget = ha.Budget(128, w["heavy"], 128)
ctxs, qs, kns, vns, outs = [], [], [], [], []
gen = torch.Generator(device=dev).manual_seed(7)
for l in range(L):
    cache = ha.PagedHashKVCache(B, 8, max(lens), dev, shuffle_seed=l)
    synthetic.fill_cache_on_device(cache, lens, seed=l)
    ctx = ha.SparseDecodeContext(cache, budget, synthetic.make_usa(32, 128, seed=l, bf16=True).packed(dev))
    ctx.hash_prefill()
    ctxs.append(ctx)
    qs.append(torch.randn(B, 32, 128, generator=gen, device=dev).bfloat16())
    kns.append(torch.randn(B, 8, 128, generator=gen, device=dev).bfloat16())
    vns.append(torch.randn(B, 8, 128, generator=gen, device=dev).bfloat16())
    outs.append(torch.empty(B, 32, 128, dtype=torch.bfloat16, device=dev))
torch.cuda.synchronize()

def capture(layers):
    g = torch.cuda.CUDAGraph(); side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for l in layers: ctxs[l].decode_step(qs[l], kns[l], vns[l], out=outs[l])
        side.synchronize()
        with torch.cuda.graph(g, stream=side):
            for l in layers: ctxs[l].decode_step(qs[l], kns[l], vns[l], out=outs[l])
    torch.cuda.current_stream().wait_stream(side)
    return g

g_all = capture(range(L)); singles = [capture([l]) for l in range(L)]
NE, NK = 6, 6
tl = torch.zeros(NK * NE * 2, dtype=torch.int64, device=dev)
names = ["hash_decode", "score_hist", "select", "gather", "merge", "select_plan"]
acc = np.zeros((NK, NE, 2))
n = 0
for rep in range(3):
    for l in range(L):
        g_all.replay(); torch.cuda.synchronize()       # makes layer l's data cold again
        init = torch.tensor([-1, 0] * (NK * NE), dtype=torch.int64, device=dev)
        tl.copy_(init); torch.cuda.synchronize()
        lib.ha_debug_set_timeline(tl.data_ptr())
        singles[l].replay(); torch.cuda.synchronize()
        lib.ha_debug_set_timeline(None)
        t = tl.cpu().numpy().astype(np.uint64).reshape(NK, NE, 2)
        t0 = t[0, 0, 0]
        acc += (t.astype(np.float64) - float(t0)) / 1000.0
        n += 1
acc /= n
print(f"{workload} B={B}: mean over {n} isolated steps, microseconds from the first CTA of hash_decode")
print(f"{'kernel':12s} {'entry min':>9s} {'entry max':>9s} {'wait min':>9s} {'wait max':>9s} {'exit min':>9s} {'exit max':>9s}   marks A/B/C (min max each, where stamped)")
for k in range(NK):
    cells = []
    for e in range(NE):
        for m in range(2):
            v = acc[k, e, m]
            cells.append(f"{v:9.2f}" if abs(v) < 1e6 else "        -")
    print(f"{names[k]:12s} " + " ".join(cells))
