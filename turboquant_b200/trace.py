"""Phase time line of one decode launch (developer tool).

    python -m turboquant_b200.trace            # config-1 shape, queries already prepared
    python -m turboquant_b200.trace --ring 100 --tokens 32768

Builds a second copy of the library with -DTQ_TRACE (every CTA of the
tensor-core decode kernel then stamps %globaltimer at its phase boundaries
into a device array), runs the decode on synthetic records and prints, for
the history CTAs, min / median / max of each stamp relative to the first CTA's
start, and for every kv head the tail of the CTA that merged it.  The trace
build is slower than the product build by the cost of the stamps; use the
numbers to see where the time goes, not as a benchmark.
"""

from __future__ import annotations

import argparse
import ctypes as C
import os
import subprocess
import sys

TRACE_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libturboquant_b200_trace.so")

STAMPS = [(0, "CTA start"), (8, "sequence length known"), (9, "block-table slice stored"), (10, "barriers ready"),
          (1, "record copies issued"), (12, "query fragments landed"), (3, "fragments + constants ready"),
          (4, "main loop done"), (5, "CTA partial written"), (6, "CTA done")]


def build_trace_lib() -> str:
    from . import build as B
    deps = B.sources() + [os.path.join(B.CSRC, f) for f in os.listdir(B.CSRC) if f.endswith(".cuh")]
    if os.path.exists(TRACE_LIB) and all(os.path.getmtime(p) <= os.path.getmtime(TRACE_LIB) for p in deps):
        return TRACE_LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *B.NVCC_FLAGS, "-DTQ_TRACE", "-I", B.INCLUDE, "-I", B.CSRC, "-o", TRACE_LIB, *B.sources()]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return TRACE_LIB


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--head-dim", type=int, default=256)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--q-heads", type=int, default=16)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--ring", type=int, default=100)
    ap.add_argument("--layers", type=int, default=8, help="pools visited round-robin so that records come from HBM")
    args = ap.parse_args()

    os.environ["TQ_B200_LIB"] = build_trace_lib()      # must be set before the library is first loaded
    import numpy as np
    import torch
    from . import _engine as E
    from . import _lib

    dev = torch.device("cuda:0")
    d, h, qh, n, ring = args.head_dim, args.kv_heads, args.q_heads, args.tokens, args.ring
    c = E.LayerConstants(d, 3, 2, dev, seed=42)
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    pools = []
    for _ in range(args.layers):
        pool = E.BlockPool(c, h, E.blocks_for(n))
        bt = E.identity_block_table(pool.num_blocks, dev)
        for pos in range(0, n, 8192):
            m = min(8192, n - pos)
            k = torch.randn(m, h, d, generator=g, device=dev).to(torch.bfloat16)
            v = torch.randn(m, h, d, generator=g, device=dev).to(torch.bfloat16)
            E.store(c, pool, k, v, stride_token=h * d, stride_head=d, n_tokens=m, n_heads=h, block_table=bt,
                    start_pos=pos)
        pools.append((pool, bt))
    rk = torch.randn(max(ring, 1), h, d, generator=g, device=dev).to(torch.bfloat16)
    rv = torch.randn(max(ring, 1), h, d, generator=g, device=dev).to(torch.bfloat16)
    rl = torch.tensor([ring], dtype=torch.int32, device=dev)
    lens = torch.tensor([n], dtype=torch.int32, device=dev)
    q = torch.randn(1, qh, d, generator=g, device=dev).to(torch.bfloat16)
    ws = E.Workspace(dev)
    splits = E.choose_splits(1, h, n, E.sm_count(dev), ring)
    n_ring = (ring + 63) // 64 if h * (splits + (ring + 63) // 64) <= E.sm_count(dev) and ring > 32 else (ring + 31) // 32
    nslot = splits + n_ring
    lib = _lib.lib()
    if not hasattr(lib, "tq_debug_read_trace"):
        raise RuntimeError("the loaded library was not built with -DTQ_TRACE")
    lib.tq_debug_read_trace.argtypes = [C.c_void_p, C.c_int]

    def run(layer: int, prepared: bool):
        pool, bt = pools[layer]
        kw = dict(ring_k=rk, ring_v=rv, ring_lens=rl, max_ring_len=ring, ring_stride_seq=0,
                  ring_stride_token=h * d) if ring > 0 else {}
        E.decode(c, pool, ws, q, bt.unsqueeze(0), lens, n, num_splits=splits, query_prepared=prepared, **kw)

    for layer in range(args.layers):
        run(layer, False)
    torch.cuda.synchronize()
    launches = 0
    for layer in range(args.layers):
        run(layer, True)
        launches += 1
        torch.cuda.synchronize()
    buf = np.zeros(4096 * 16, dtype=np.uint64)
    lib.tq_debug_read_trace(buf.ctypes.data, buf.size)
    ncta = nslot * h
    # the library alternates between two trace slots per launch; the last launch's slot holds the newest stamps
    slots = buf.reshape(2, 2048, 16)[:, :ncta].astype(np.int64)
    t = slots[int(np.argmax([s[:, 0].min() for s in slots]))]
    x = np.arange(ncta) // h            # CTA index = kv head + H * slot
    hist, rg = t[x < splits], t[x >= splits]
    t0 = t[:, 0].min()

    def fmt(a):
        return f"min {a.min() / 1e3:6.2f}  med {np.median(a) / 1e3:6.2f}  max {a.max() / 1e3:6.2f}"

    print(f"head_dim {d}, {h} kv heads, {qh} query heads, {n} tokens, ring {ring}: {splits} history + {n_ring} ring CTAs "
          f"per kv head, {ncta} CTAs; times in us after the first CTA's start")
    for idx, name in STAMPS:
        print(f"  {name:30s} {fmt(hist[:, idx] - t0)}")
    if len(rg):
        print(f"  {'ring CTAs: partial written':30s} {fmt(rg[:, 5] - t0)}")
    for hh in range(h):
        blk = t[hh::h]
        i = int(np.argmax(blk[:, 6]))
        print(f"  kv head {hh}: merged by CTA {i}: partial written {(blk[i, 5] - t0) / 1e3:6.2f}, ticket known "
              f"{(blk[i, 7] - t0) / 1e3:6.2f}, partials landed {(blk[i, 13] - t0) / 1e3:6.2f}, max known "
              f"{(blk[i, 14] - t0) / 1e3:6.2f}, slots summed {(blk[i, 15] - t0) / 1e3:6.2f}, output written "
              f"{(blk[i, 6] - t0) / 1e3:6.2f}")
    print(f"  launch span {(t[:, 6].max() - t0) / 1e3:6.2f} us")
    sys.stdout.flush()


if __name__ == "__main__":
    main()
