#!/usr/bin/env python
"""Benchmark of the TurboQuant KV-cache hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: decode attention of one long sequence shaped like a
hybrid model's full-attention layer - head_dim 256, 4 kv heads, 16 query heads,
32768 compressed tokens (3-bit keys, 2-bit values), bf16, plus an exact bf16 ring
of up to 128 recent tokens.  A step = append one new token through the store
path (ring write; a full ring is compressed into the store as one 128-token
chunk) + one decode-attention call.  The steps rotate over 8 independent layers
so that the bytes touched between two visits of a layer (8 x 25.8 MB) exceed the
126 MB L2: every step streams its compressed history from HBM.

`value` is KV tokens attended per second with everything resident in HBM (steps
replayed from CUDA graphs); `e2e` is the same metric through the Python API with
pinned host buffers: every step moves the new key/value/query to the device and the
attention output back inside the timed region.  With N > 1 every rank runs
its own sequences (weak scaling, no data-path collective) and the time is the max
over ranks.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WL = dict(name="config1: decode D=256 Hkv=4 Hq=16 N=32768 ring=128 key3b/val2b bf16",
          D=256, H=4, Qh=16, N=32768, ring=128, key_bits=3, value_bits=2, layers=8)
METRIC = "decode_attention_kv_tokens_per_s"
UNIT = "tokens/s"
N_NEW = 256  # distinct new tokens / queries per layer, reused cyclically
# Files whose contents decide what the decode kernel reads and writes: the recorded DRAM traffic of a
# launch is only quoted while they are unchanged since the capture.
TRAFFIC_RECORD = os.path.join(ROOT, "profiles", "decode_traffic.json")
TRAFFIC_SOURCES = ("turboquant_b200/csrc/tq_decode_mma.cu", "turboquant_b200/csrc/tq_decode_common.cuh",
                   "turboquant_b200/csrc/tq_common.cuh")


def sources_digest() -> str:
    import hashlib
    hsh = hashlib.sha256()
    for rel in TRAFFIC_SOURCES:
        with open(os.path.join(ROOT, rel), "rb") as fh:
            hsh.update(fh.read())
    return hsh.hexdigest()[:16]


def recorded_traffic():
    """(bytes per launch, note): dram__bytes_read.sum + dram__bytes_write.sum of one decode launch of the
    headline workload from the last ncu capture, or (None, why) when the kernel's sources changed since."""
    try:
        with open(TRAFFIC_RECORD) as fh:
            rec = json.load(fh)
    except (OSError, ValueError):
        return None, "no ncu capture recorded"
    if rec.get("sources_digest") != sources_digest():
        return None, "kernel sources changed since the recorded ncu capture"
    return float(rec["dram_bytes_per_launch"]), rec.get("source", "ncu capture")


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the GPU works."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------------------
# CUDA arm
# --------------------------------------------------------------------------------------

class Layer:
    """One layer's compressed store, exact ring and synthetic token stream."""

    def __init__(self, idx: int, rank: int, dev):
        from turboquant_b200 import CompressedKVStore
        w = WL
        self.store = CompressedKVStore(w["D"], w["H"], w["key_bits"], w["value_bits"], device=dev, layer_idx=idx,
                                       capacity_tokens=w["N"] + 64 * w["ring"])
        g = torch.Generator(device=dev)
        g.manual_seed(1001 + 97 * rank + idx)
        ch = torch.exp(0.5 * torch.randn(w["D"], generator=g, device=dev))
        shape = (w["H"], w["D"])
        for pos in range(0, w["N"], 8192):
            n = min(8192, w["N"] - pos)
            k = (torch.randn(n, *shape, generator=g, device=dev) * ch).to(torch.bfloat16)
            v = torch.randn(n, *shape, generator=g, device=dev).to(torch.bfloat16)
            self.store.append_chunk(k, v)
        self.new_k = (torch.randn(N_NEW, *shape, generator=g, device=dev) * ch).to(torch.bfloat16)
        self.new_v = torch.randn(N_NEW, *shape, generator=g, device=dev).to(torch.bfloat16)
        self.query = torch.randn(N_NEW, 1, w["Qh"], w["D"], generator=g, device=dev).to(torch.bfloat16)
        self.ring_k = (torch.randn(w["ring"], *shape, generator=g, device=dev) * ch).to(torch.bfloat16)
        self.ring_v = torch.randn(w["ring"], *shape, generator=g, device=dev).to(torch.bfloat16)
        # staggered fill so that ring flushes are spread over the run at their natural rate
        self.ring_pos = w["ring"] - 16 * idx
        self.ring_len = torch.full((1,), self.ring_pos, dtype=torch.int32, device=dev)
        self.out = torch.empty(1, w["Qh"], w["D"], dtype=torch.bfloat16, device=dev)
        self.steps = 0


class Runner:
    def __init__(self, rank: int, dev):
        from turboquant_b200 import _engine as E
        self.E, self.dev = E, dev
        self.layers = [Layer(i, rank, dev) for i in range(WL["layers"])]
        self.splits = E.choose_splits(1, WL["H"], WL["N"], E.sm_count(dev), WL["ring"])
        self.launches = 0      # kernels of this library
        self.tokens = 0        # KV tokens attended
        self.bytes = 0         # algorithmic bytes of the decode kernel

    def decode(self, L: Layer, q, prepared=False, append=None):
        E, w = self.E, WL
        kw = {}
        if append is not None:       # the new token is written into the ring by the decode call itself
            kw = dict(append_k=append[0], append_v=append[1])
        E.decode(L.store.consts, L.store.pool, L.store.workspace, q, L.store.block_table.unsqueeze(0),
                 L.store.seq_len_device, L.store.num_tokens, ring_k=L.ring_k, ring_v=L.ring_v, ring_lens=L.ring_len,
                 max_ring_len=L.ring_pos, ring_stride_seq=0, ring_stride_token=w["H"] * w["D"],
                 num_splits=self.splits, out=L.out, query_prepared=prepared, **kw)
        self.launches += 1 if prepared else 2
        self.tokens += L.store.num_tokens + L.ring_pos
        self.bytes += self.decode_bytes(L)

    @staticmethod
    def decode_bytes(L: Layer) -> int:
        w = WL
        return L.store.memory_bytes() + L.ring_pos * w["H"] * w["D"] * 2 * 2

    def step(self, s: int):
        """Global step s: layer s % L appends a token and decodes."""
        w = WL
        L = self.layers[s % w["layers"]]
        i = L.steps % N_NEW
        if L.ring_pos >= w["ring"]:                      # ring full: compress it as one chunk
            L.store.append_chunk(L.ring_k, L.ring_v)
            self.launches += 1
            L.ring_pos = 0
            L.ring_len.zero_()
        L.ring_pos += 1                                  # device side: ring_len += 1 inside the decode call
        self.decode(L, L.query[i], append=(L.new_k[i:i + 1], L.new_v[i:i + 1]))
        L.steps += 1

    def capture(self, first: int, count: int, chunk: int = 256):
        """CUDA graphs replaying steps [first, first+count); host state advances now."""
        graphs = []
        s = first
        while s < first + count:
            n = min(chunk, first + count - s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for j in range(s, s + n):
                    self.step(j)
            graphs.append(g)
            s += n
        return graphs


def _dist():
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    if ws > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
        return dist, dist.get_rank(), ws
    return None, 0, 1


def measure_store(dev):
    """Prefill store throughput: 131072 tokens of one sequence appended in 16 chunks of 8192, 8 kv heads,
    head_dim 128, bf16, 3-bit keys / 2-bit values, written into 16-token block records through a shuffled
    block table.  The 16 store calls are captured in one CUDA graph and replayed (device time of the whole
    run: 537 MB of input, larger than L2); the same run through CompressedKVStore.append_chunk, launched
    eagerly from Python, is reported beside it."""
    from turboquant_b200 import CompressedKVStore, _engine as E
    t, h, d, chunks = 8192, 8, 128, 16
    n = t * chunks
    c = E.LayerConstants(d, 3, 2, dev, seed=42)
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    ch = torch.exp(0.5 * torch.randn(d, generator=g, device=dev))
    k = (torch.randn(n, h, d, generator=g, device=dev) * ch).to(torch.bfloat16)
    v = torch.randn(n, h, d, generator=g, device=dev).to(torch.bfloat16)
    nb = n // 16
    pool = E.BlockPool(c, h, nb)
    bt = torch.randperm(nb, generator=torch.Generator().manual_seed(4)).int().to(dev)

    def run():
        for i in range(chunks):
            E.store(c, pool, k[i * t:(i + 1) * t], v[i * t:(i + 1) * t], stride_token=h * d, stride_head=d, n_tokens=t,
                    n_heads=h, block_table=bt, start_pos=i * t)

    run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    graph.replay()
    torch.cuda.synchronize()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms_run = e0.elapsed_time(e1) / reps
    status = E.store_status()
    st = CompressedKVStore(d, h, 3, 2, device=dev, capacity_tokens=n)
    st.append_chunk(k[:t], v[:t])
    st.reset()
    torch.cuda.synchronize()
    e0.record()
    for i in range(chunks):
        st.append_chunk(k[i * t:(i + 1) * t], v[i * t:(i + 1) * t])
    e1.record()
    torch.cuda.synchronize()
    ms_api = e0.elapsed_time(e1)
    nbytes = n * h * (2 * d * 2 + c.bytes_per_token)
    peak, kind = _peaks()
    tflops = 6 * 2 * 128.0 * 128 * n * h / (ms_run * 1e-3) / 1e12      # six 128-wide bf16 products per token-head
    return {"workload": "131072 tok in 16 chunks of 8192 x 8 heads x 128 bf16, key3b/val2b, paged block records",
            "ms_per_run": ms_run, "ms_per_chunk": ms_run / chunks, "gbs": nbytes / ms_run / 1e6,
            "frac": nbytes / ms_run / 1e6 / peak, "peak_kind": f"of {kind}", "tensor_tflops": tflops,
            "token_heads_per_s": n * h / ms_run * 1e3, "api_ms_per_chunk": ms_api / chunks,
            "api_gbs": nbytes / ms_api / 1e6, "device_status": status}


def measure_prefill(dev):
    """Causal prefill attention of the no-alloc mode (the layer's own K/V, no paged cache) followed by the
    store of the same K/V: one 8192-token sequence, 32 query heads over 8 kv heads, head_dim 128, bf16.  The
    attention kernel is tensor-bound: flops = 4 * n^2 / 2 * D * Qh against the measured bf16 matmul peak."""
    from turboquant_b200 import CompressedKVStore, _engine as E
    n, qh, h, d = 8192, 32, 8, 128
    g = torch.Generator(device=dev)
    g.manual_seed(8)
    q = torch.randn(n, qh, d, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(n, h, d, generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn(n, h, d, generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    st = CompressedKVStore(d, h, 3, 2, device=dev, capacity_tokens=n)

    def step(with_store):
        E.prefill_attention(q, k, v, out=out)
        if with_store:
            st.reset()
            st.append_chunk(k, v)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ms = {}
    for with_store in (False, True):
        for _ in range(3):
            step(with_store)
        torch.cuda.synchronize()
        reps = 10
        e0.record()
        for _ in range(reps):
            step(with_store)
        e1.record()
        torch.cuda.synchronize()
        ms[with_store] = e0.elapsed_time(e1) / reps
    flops = 4.0 * n * n / 2 * d * qh
    peak_tf = 1590.0
    kind = "fallback"
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            peak_tf, kind = float(json.load(fh)["bf16_tflops"]), "measured"
    tf = flops / (ms[False] * 1e-3) / 1e12
    return {"workload": "causal prefill attention, 8192 tokens, 32 query / 8 kv heads, D=128, bf16", "ms_attention": ms[False],
            "ms_attention_and_store": ms[True], "tflops": tf,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf,
                         "peak_kind": f"of {kind} (burst)"},
            "device_status": E.prefill_attention_status()}


def measure_decode_large(dev, n_seq: int = 256, n_tok: int = 8192):
    """Batched decode of one Llama-3-70B-shaped layer: 256 sequences x
    8192 compressed tokens, 8 kv heads, 64 query heads, head_dim 128, 3-bit keys / 2-bit values.
    1.68 GB of compressed records per launch: fixed launch costs are amortised, which shows
    what the kernel itself streams."""
    from turboquant_b200 import _engine as E
    d, h, qh = 128, 8, 64
    c = E.LayerConstants(d, 3, 2, dev, seed=42)
    nblk = n_tok // 16
    pool = E.BlockPool(c, h, n_seq * nblk)
    bt = torch.arange(n_seq * nblk, dtype=torch.int32, device=dev).view(n_seq, nblk)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    ch = torch.exp(0.5 * torch.randn(d, generator=g, device=dev))
    for s in range(n_seq):
        k = (torch.randn(n_tok, h, d, generator=g, device=dev) * ch).to(torch.bfloat16)
        v = torch.randn(n_tok, h, d, generator=g, device=dev).to(torch.bfloat16)
        E.store(c, pool, k, v, stride_token=h * d, stride_head=d, n_tokens=n_tok, n_heads=h, block_table=bt[s],
                start_pos=0)
    q = torch.randn(n_seq, qh, d, generator=g, device=dev).to(torch.bfloat16)
    lens = torch.full((n_seq,), n_tok, dtype=torch.int32, device=dev)
    ws = E.Workspace(dev)
    out = torch.empty_like(q)
    for _ in range(3):
        E.decode(c, pool, ws, q, bt, lens, n_tok, out=out)
    torch.cuda.synchronize()
    ms, ms_step = _time_decode(lambda prepared: E.decode(c, pool, ws, q, bt, lens, n_tok, out=out,
                                                         query_prepared=prepared))
    nbytes = n_seq * n_tok * h * c.bytes_per_token
    peak, kind = _peaks()
    return {"workload": f"config4 layer: {n_seq} seqs x {n_tok} tok, Hkv=8 Hq=64 D=128 key3b/val2b",
            "ms_per_launch": ms, "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak, "peak_kind": f"of {kind}",
            "ms_per_step_with_query_prep": ms_step, "frac_with_query_prep": nbytes / ms_step / 1e6 / peak,
            "kv_tokens_per_s": n_seq * n_tok / ms_step * 1e3, "device_status": ws.status()}


def _time_decode(call, reps: int = 10):
    """(ms per decode launch with the query already prepared, ms per step including query preparation)."""
    out = []
    for prepared in (True, False):
        call(False)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            call(prepared)
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / reps)
    return out[0], out[1]


def measure_decode_paged(dev, n_seq: int = 64, lo: int = 1024, hi: int = 32768):
    """Batched paged decode: 64 sequences of length U[1024, 32768], block size 16, head_dim 128,
    8 kv heads, 32 query heads, bf16, 4-bit keys (3-bit codes + QJL sign) and 4-bit values, one query per sequence,
    block tables = a seeded random permutation of a shared pool."""
    from turboquant_b200 import _engine as E
    d, h, qh = 128, 8, 32
    c = E.LayerConstants(d, 4, 4, dev, seed=42)
    gcpu = torch.Generator().manual_seed(11)
    lens_l = [int(x) for x in torch.randint(lo, hi + 1, (n_seq,), generator=gcpu)]
    per = [(n + 15) // 16 for n in lens_l]
    total = sum(per)
    perm = torch.randperm(total, generator=gcpu).to(torch.int32)
    bt = torch.zeros(n_seq, max(per), dtype=torch.int32)
    pos = 0
    for s_, nb in enumerate(per):
        bt[s_, :nb] = perm[pos:pos + nb]
        pos += nb
    bt = bt.to(dev)
    pool = E.BlockPool(c, h, total)
    g = torch.Generator(device=dev)
    g.manual_seed(6)
    ch = torch.exp(0.5 * torch.randn(d, generator=g, device=dev))
    for s_ in range(n_seq):
        n = lens_l[s_]
        k = (torch.randn(n, h, d, generator=g, device=dev) * ch).to(torch.bfloat16)
        v = torch.randn(n, h, d, generator=g, device=dev).to(torch.bfloat16)
        E.store(c, pool, k, v, stride_token=h * d, stride_head=d, n_tokens=n, n_heads=h, block_table=bt[s_],
                start_pos=0)
    q = torch.randn(n_seq, qh, d, generator=g, device=dev).to(torch.bfloat16)
    lens = torch.tensor(lens_l, dtype=torch.int32, device=dev)
    ws = E.Workspace(dev)
    out = torch.empty_like(q)
    for _ in range(3):
        E.decode(c, pool, ws, q, bt, lens, max(lens_l), out=out)
    torch.cuda.synchronize()
    ms, ms_step = _time_decode(lambda prepared: E.decode(c, pool, ws, q, bt, lens, max(lens_l), out=out,
                                                         query_prepared=prepared))
    nbytes = sum(lens_l) * h * c.bytes_per_token
    peak, kind = _peaks()
    return {"workload": f"config2: {n_seq} seqs x U[{lo},{hi}] tok paged, Hkv=8 Hq=32 D=128 key4b/val4b",
            "ms_per_launch": ms, "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak, "peak_kind": f"of {kind}",
            "ms_per_step_with_query_prep": ms_step, "frac_with_query_prep": nbytes / ms_step / 1e6 / peak,
            "kv_tokens_per_s": sum(lens_l) / ms_step * 1e3, "device_status": ws.status()}


def measure_sharded(dev, dist, rank: int, world: int, layers: int = 8, reps: int = 5):
    """A stack of Llama-3-70B-shaped attention layers (256 sequences x 8192 compressed tokens, 8 kv heads,
    64 query heads, head_dim 128, 3-bit keys / 2-bit values) partitioned over the ranks - sequences first -
    with an all-gather of the head outputs (NCCL) per layer.  Total work is fixed (strong scaling).  A step =
    every layer once: query preparation + decode written straight into the rank's band of the full output,
    then the gather (a) serialised behind the decode on the same stream and (b) on a second stream, under
    the decode of the next layer.  Times are CUDA events, max over ranks."""
    from turboquant_b200 import _engine as E
    from turboquant_b200 import sharding
    d, h, qh, n_seq, n_tok = 128, 8, 64, 256, 8192
    sh = sharding.partition(n_seq, h, world, rank)
    hl, sl = sh.num_heads, sh.num_seqs
    g_heads = qh // h
    nblk = n_tok // 16
    consts, pools, queries, outs = [], [], [], []
    bt = torch.arange(sl * nblk, dtype=torch.int32, device=dev).view(sl, nblk)
    g = torch.Generator(device=dev)
    for layer in range(layers):
        c = E.LayerConstants(d, 3, 2, dev, seed=42 + 7 * layer)
        pool = E.BlockPool(c, hl, sl * nblk)
        g.manual_seed(100003 * layer + 17 * rank + 1)      # one stream per (layer, shard): ranks build locally
        ch = torch.exp(0.5 * torch.randn(d, generator=g, device=dev))
        for s0 in range(0, sl, 16):
            ns = min(16, sl - s0)
            k = (torch.randn(ns, n_tok, hl, d, generator=g, device=dev) * ch).to(torch.bfloat16)
            v = torch.randn(ns, n_tok, hl, d, generator=g, device=dev).to(torch.bfloat16)
            for j in range(ns):
                E.store(c, pool, k[j], v[j], stride_token=hl * d, stride_head=d, n_tokens=n_tok, n_heads=hl,
                        block_table=bt[s0 + j], start_pos=0)
        consts.append(c)
        pools.append(pool)
        queries.append(torch.randn(sl, hl * g_heads, d, generator=g, device=dev).to(torch.bfloat16))
        outs.append(torch.empty(n_seq, qh, d, dtype=torch.bfloat16, device=dev))
    lens = torch.full((sl,), n_tok, dtype=torch.int32, device=dev)
    ws = E.Workspace(dev)
    slabs = [sharding.output_slab(o, sh, h) for o in outs]
    in_place = all(x is not None for x in slabs)
    if not in_place:
        slabs = [torch.empty(sl, hl * g_heads, d, dtype=torch.bfloat16, device=dev) for _ in outs]
    comm = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)

    def decode(layer):
        E.decode(consts[layer], pools[layer], ws, queries[layer], bt, lens, n_tok, out=slabs[layer])

    def gather(layer):
        sharding.gather_head_outputs(slabs[layer], sh, n_seq, h, out=outs[layer])

    def step_serial():
        for layer in range(layers):
            decode(layer)
            gather(layer)

    def step_overlap():
        for layer in range(layers):
            decode(layer)
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                gather(layer)
        main.wait_stream(comm)

    def step_local():
        for layer in range(layers):
            decode(layer)

    def step_gather_only():
        for layer in range(layers):
            gather(layer)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if dist is not None:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    ms_local = timed(step_local)
    ms_serial = timed(step_serial) if world > 1 else ms_local
    ms_overlap = timed(step_overlap) if world > 1 else ms_local
    ms_gather = timed(step_gather_only) if world > 1 else 0.0
    status = ws.status()
    nbytes = layers * n_seq * n_tok * h * consts[0].bytes_per_token
    peak, kind = _peaks()
    return {"workload": f"{layers} layers x 256 seqs x 8192 tok, Hkv=8 Hq=64 D=128 key3b/val2b (fixed total: strong scaling)",
            "partition": f"sequences first: {sl} sequences x {hl} kv heads per rank", "layers": layers,
            "collective": "all-gather of head outputs per layer (torch.distributed, NCCL), received in place",
            "gathered_bytes_per_layer": n_seq * qh * d * 2,
            "ms_per_step_decode_only": ms_local, "ms_per_step_serialised": ms_serial, "ms_per_step_overlapped": ms_overlap,
            "allgather_us_per_layer": ms_gather / layers * 1e3,
            "ms_per_layer_overlapped": ms_overlap / layers,
            "kv_tokens_per_s": layers * n_seq * n_tok / ms_overlap * 1e3,
            "aggregate_hbm_gbs": nbytes / ms_overlap / 1e6, "frac_per_gpu": nbytes / ms_overlap / 1e6 / world / peak,
            "peak_kind": f"of {kind}", "timing": "CUDA events, max over ranks", "device_status": status}


def run_sharded(args):
    """`--sharded`: only the partitioned layer stack (see measure_sharded)."""
    dist, rank, world = _dist()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    res = measure_sharded(dev, dist, rank, world)
    if rank == 0:
        print(json.dumps({"metric": "sharded_layer_stack_decode_kv_tokens_per_s", "value": res["kv_tokens_per_s"],
                          "unit": UNIT, "n_gpus": world, "ms_per_step": res["ms_per_step_overlapped"],
                          "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": res["workload"]}, "sharded": res}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def cpu_baseline(steps: int, warmup: int, n_hist: int):
    """The oracle (a torch-CPU restatement of the reference's path) on the host cores."""
    # all host threads the process may use, whatever OMP_NUM_THREADS the launcher exported (torchrun sets 1)
    try:
        n_cpu = len(os.sched_getaffinity(0))
    except AttributeError:
        n_cpu = os.cpu_count() or 1
    torch.set_num_threads(max(1, n_cpu))
    from oracle import tq_oracle as O
    from turboquant_b200.codebook import get_codebook_tensors
    w = WL
    cent, bnd = get_codebook_tensors(w["D"], w["key_bits"] - 1, "cpu")
    st = O.OracleStore(w["D"], w["H"], w["key_bits"], w["value_bits"], cent, bnd, layer_idx=0)
    k, v = O.synth_kv(n_hist + w["ring"] + steps + warmup + 1, w["H"], w["D"], seed=1001, dtype=torch.bfloat16)
    q = O.synth_query(steps + warmup + 1, w["Qh"], w["D"], seed=7, dtype=torch.bfloat16)
    t0 = time.perf_counter()
    for pos in range(0, n_hist, 8192):
        st.append_chunk(k[pos:pos + 8192][: n_hist - pos], v[pos:pos + 8192][: n_hist - pos])
    store_s = time.perf_counter() - t0
    ring_k, ring_v = [k[n_hist:n_hist + w["ring"]]], [v[n_hist:n_hist + w["ring"]]]
    ring_n = w["ring"]
    tokens, t_start = 0, None
    for s in range(warmup + steps):
        if s == warmup:
            t_start, tokens = time.perf_counter(), 0
        if ring_n >= w["ring"]:      # flush the ring as one chunk (capture.py:89-96)
            st.append_chunk(torch.cat(ring_k), torch.cat(ring_v))
            ring_k, ring_v, ring_n = [], [], 0
        i = n_hist + w["ring"] + s
        ring_k.append(k[i:i + 1])
        ring_v.append(v[i:i + 1])
        ring_n += 1
        flat = st.get_flat_cache()
        O.hybrid_attention(q[s:s + 1], flat, torch.cat(ring_k), torch.cat(ring_v), w["H"], st.pi, st.s, cent)
        tokens += flat.num_tokens + ring_n
    dt = time.perf_counter() - t_start
    return {"value": tokens / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{steps} full decode steps over {n_hist} compressed tokens + ring on the host CPU "
                      f"(torch {torch.__version__}); store of the history took {store_s:.2f} s "
                      f"= {n_hist * w['H'] / store_s:.0f} token-heads/s",
            "ms_per_step": dt / steps * 1e3}


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:   # under torchrun only rank 0 measures the host CPU
        return
    n_hist = WL["N"] if args.steps <= 100 else 8192
    base = cpu_baseline(args.steps, args.warmup, n_hist)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WL["name"], "history_tokens_per_step": n_hist,
                       "note": "reference path = dequantise all history to fp32, then einsum/softmax/einsum on CPU"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_ours(args):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this path has no CPU fallback")
    dist, rank, world = _dist()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    w = WL
    sampler = ClockSampler(local)

    runner = Runner(rank, dev)
    nl = w["layers"]
    for s in range(nl):                      # eager pass: sizes workspaces, sets kernel attributes
        runner.step(s)
    torch.cuda.synchronize()
    warm = runner.capture(nl, args.warmup)
    runner.launches = runner.tokens = runner.bytes = 0
    timed = runner.capture(nl + args.warmup, args.steps)
    launches, tokens, dec_bytes = runner.launches, runner.tokens, runner.bytes

    sampler.start()
    for g in warm:
        g.replay()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for g in timed:
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    agg_tokens = tokens
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        tk = torch.tensor([float(tokens)], device=dev, dtype=torch.float64)
        dist.all_reduce(tk)
        agg_tokens = float(tk.item())
    status = max(L.store.workspace.status() for L in runner.layers)

    # ---- roofline of the decode kernel: decode-only launches, queries already prepared ----
    reps = 8
    for L in runner.layers:
        runner.decode(L, L.query[0])
    runner.bytes = 0
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for r in range(reps):
            for L in runner.layers:
                runner.decode(L, L.query[0], prepared=True)
    bytes_per_launch = runner.bytes / (reps * nl)
    g.replay()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(5):
        g.replay()
    k1.record()
    torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / (5 * reps * nl)
    peak, peak_kind = _peaks()
    achieved = bytes_per_launch / kern_ms / 1e6
    traffic, traffic_note = recorded_traffic()

    # ---- end to end through the Python API with host buffers ----
    from turboquant_b200 import KVCaptureEngine, compute_hybrid_attention
    e2e_steps = max(8, min(args.steps, 256))
    engines = []
    for L in runner.layers:
        eng = KVCaptureEngine(L.store, ring_capacity=w["ring"], device=dev)
        eng.ring.write(L.ring_k[:L.ring_pos], L.ring_v[:L.ring_pos], L.ring_pos)
        engines.append(eng)
    H, Qh, D = w["H"], w["Qh"], w["D"]
    nk, nq = H * D, Qh * D
    # one pinned host row per new token: key | value | query, moved with ONE copy per step
    hpack = torch.randn(N_NEW, 2 * nk + nq).to(torch.bfloat16).pin_memory()
    hout = torch.empty(1, Qh, D, dtype=torch.bfloat16).pin_memory()
    dstage = torch.empty(2 * nk + nq, dtype=torch.bfloat16, device=dev)
    dk, dv = dstage[:nk].view(1, H, D), dstage[nk:2 * nk].view(1, H, D)
    dq = dstage[2 * nk:].view(1, Qh, D)
    dout = torch.empty(1, Qh, D, dtype=torch.bfloat16, device=dev)

    def e2e_step(s):
        """The fused call: ring append + attention in one library call."""
        eng = engines[s % nl]
        dstage.copy_(hpack[s % N_NEW], non_blocking=True)
        eng.decode_step(dq, dk, dv, Qh, out=dout)
        hout.copy_(dout, non_blocking=True)
        return eng.total_tokens

    def e2e_step_host(s):
        """Host buffers in, host buffer out: copies, ring append and attention enqueued by one library call."""
        eng = engines[s % nl]
        eng.decode_step_host(hpack[s % N_NEW], hout.view(-1), Qh)
        return eng.total_tokens

    def e2e_step_two_calls(s):
        """The reference's call sequence: ingest_decode, then compute_hybrid_attention."""
        eng = engines[s % nl]
        dstage.copy_(hpack[s % N_NEW], non_blocking=True)
        eng.ingest_decode(dk, dv, 1)
        rk, rv = eng.ring.peek()
        out = compute_hybrid_attention(dq, eng.store, rk, rv, Qh)
        hout.copy_(out, non_blocking=True)
        return eng.total_tokens

    def run_e2e(step_fn, first):
        for s in range(first, first + nl):
            step_fn(s)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        toks = 0
        t0 = time.perf_counter()
        for s in range(first + nl, first + nl + e2e_steps):
            toks += step_fn(s)
        torch.cuda.synchronize()
        secs = time.perf_counter() - t0
        if dist is not None:
            t = torch.tensor([secs], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            secs = float(t.item())
            tk = torch.tensor([float(toks)], device=dev, dtype=torch.float64)
            dist.all_reduce(tk)
            toks = float(tk.item())
        return toks, secs

    two_tokens, two_s = run_e2e(e2e_step_two_calls, 0)
    fused_tokens, fused_s = run_e2e(e2e_step, nl + e2e_steps)
    e2e_tokens, e2e_s = run_e2e(e2e_step_host, 2 * (nl + e2e_steps))
    # the same call with the stream synchronised after every step: what a caller sees who needs the
    # output of step i before it can issue step i+1
    sync_n = min(e2e_steps, 64)
    t0 = time.perf_counter()
    for s in range(3 * (nl + e2e_steps), 3 * (nl + e2e_steps) + sync_n):
        e2e_step_host(s)
        torch.cuda.synchronize()
    synced_ms = (time.perf_counter() - t0) / sync_n * 1e3
    clocks = sampler.stop()

    sharded = measure_sharded(dev, dist, rank, world) if not args.no_large else None   # every rank takes part
    def extra(fn, *a):
        """A secondary measurement (rank 0 only, no collective inside): its failure is reported in its key
        instead of taking the headline line down with it."""
        try:
            return fn(*a)
        except Exception as exc:      # noqa: BLE001 - the line must still be printed
            torch.cuda.synchronize()
            return {"error": f"{type(exc).__name__}: {exc}"[:300]}

    store = extra(measure_store, dev) if rank == 0 else None
    prefill = extra(measure_prefill, dev) if (rank == 0 and not args.no_large) else None
    large = extra(measure_decode_large, dev) if (rank == 0 and not args.no_large) else None
    paged = extra(measure_decode_paged, dev) if (rank == 0 and not args.no_large) else None
    base = extra(cpu_baseline, 3, 1, w["N"]) if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None

    if rank == 0:
        line = {
            "metric": METRIC, "value": agg_tokens / ms * 1e3, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "layers_rotating": nl,
                       "l2": "inputs larger than L2: 8 layers x 25.8 MB compressed history visited round-robin",
                       "splits_per_kv_head": runner.splits, "steps_replayed_from": "CUDA graphs",
                       "parallelism": f"dp{world} (independent sequences per GPU, no collective on the data path)"},
            "hbm_gbs": dec_bytes / ms / 1e6 * world,
            "roofline": {"bound": "hbm", "kernel": "tq_decode_mma_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "frac_of_nominal_8TBs": achieved / 8000.0, "us_per_launch": kern_ms * 1e3,
                         "bytes_per_launch": bytes_per_launch, "traffic": traffic, "traffic_source": traffic_note},
            "e2e": {"value": e2e_tokens / e2e_s, "unit": UNIT, "steps": e2e_steps,
                    "ms_per_step": e2e_s / e2e_steps * 1e3, "synced_ms_per_step": synced_ms,
                    "call": "KVCaptureEngine.decode_step_host (pinned host buffers; H2D copy, ring append + attention, "
                            "D2H copy enqueued by one library call)",
                    "device_tensor_call_value": fused_tokens / fused_s,
                    "device_tensor_call_ms_per_step": fused_s / e2e_steps * 1e3,
                    "device_tensor_call": "torch H2D copy + KVCaptureEngine.decode_step + torch D2H copy",
                    "two_call_value": two_tokens / two_s, "two_call_ms_per_step": two_s / e2e_steps * 1e3,
                    "two_call": "ingest_decode + compute_hybrid_attention (the reference's call sequence)",
                    "h2d_bytes_per_step": (2 * w["H"] + w["Qh"]) * w["D"] * 2,
                    "d2h_bytes_per_step": w["Qh"] * w["D"] * 2},
            "gpu_launches": launches, "device_status": status, "clocks": clocks, "store": store,
            "decode_large": large, "decode_paged": paged, "sharded": sharded, "prefill": prefill,
        }
        if base is not None:
            line["cpu_baseline"] = base if "error" in base else {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-large", action="store_true", help="skip the batched 1.7 GB decode measurement")
    ap.add_argument("--only-large", action="store_true", help="run only the batched decode measurement (profiling)")
    ap.add_argument("--only-store", action="store_true", help="run only the store-path measurement (profiling)")
    ap.add_argument("--only-paged", action="store_true", help="run only the paged batched decode measurement (profiling)")
    ap.add_argument("--only-prefill", action="store_true", help="run only the prefill attention measurement (profiling)")
    ap.add_argument("--sharded", action="store_true",
                    help="only the partitioned layer stack with its all-gather of head outputs (strong scaling)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.only_store:
        torch.cuda.set_device(0)
        print(json.dumps(measure_store(torch.device("cuda", 0))), flush=True)
    elif args.only_prefill:
        torch.cuda.set_device(0)
        print(json.dumps(measure_prefill(torch.device("cuda", 0))), flush=True)
    elif args.only_paged:
        torch.cuda.set_device(0)
        print(json.dumps(measure_decode_paged(torch.device("cuda", 0))), flush=True)
    elif args.only_large:
        torch.cuda.set_device(0)
        print(json.dumps(measure_decode_large(torch.device("cuda", 0))), flush=True)
    elif args.sharded:
        run_sharded(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
