"""Generate the golden fixtures in this directory by running the reference.

Run once in the build container, where the reference tree is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference package, redirects its code-book cache to a scratch
directory (the reference otherwise writes missing code books into its own
package directory, codebook.py:158-170), executes the reference's store and
read paths on small seeded inputs and writes one .npz per case.  The tests
only read the .npz files; they never need the reference tree.

Every case stores its inputs, the per-layer constants (Pi, S, code book) and
every intermediate of the key path, so each stage can be checked alone.
bf16 tensors are stored as uint16 bit patterns (suffix `_bf16`).
"""

from __future__ import annotations

import os
import shutil
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [
    # name, D, H, Qh, T, ring, dtype, key_bits, value_bits, layer_idx, input seed
    ("d128_fp32_k3v2", 128, 2, 8, 80, 24, torch.float32, 3, 2, 0, 1000),
    ("d128_bf16_k3v2", 128, 2, 8, 80, 24, torch.bfloat16, 3, 2, 0, 1001),
    ("d256_bf16_k3v2", 256, 2, 8, 48, 16, torch.bfloat16, 3, 2, 1, 1002),
    ("d128_bf16_k4v4", 128, 2, 8, 64, 8, torch.bfloat16, 4, 4, 2, 1003),
    ("d128_fp16_k3v2", 128, 1, 4, 32, 4, torch.float16, 3, 2, 0, 1004),
]


def _np(t: torch.Tensor):
    """(array, key suffix) for a tensor; bf16 travels as uint16 bits."""
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), "_bf16"
    return t.numpy(), ""


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import turboquant  # noqa: F401  (the reference)
    import turboquant.codebook as ref_codebook
    from turboquant.kv_cache import quantize_values
    from turboquant.rotation import rotate_forward
    from turboquant.score import compute_hybrid_attention
    from turboquant.store import CompressedKVStore

    scratch = tempfile.mkdtemp(prefix="tq_codebooks_")
    for f in os.listdir(ref_codebook._CODEBOOK_DIR):
        if f.endswith(".json"):
            shutil.copy(os.path.join(ref_codebook._CODEBOOK_DIR, f), scratch)
    ref_codebook._CODEBOOK_DIR = scratch

    cpu = torch.device("cpu")
    for name, d, h, qh, t, ring, dtype, kb, vb, layer, seed in CASES:
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)
        ch = torch.exp(0.5 * torch.randn(d, generator=g))
        key = (torch.randn(t + ring, h, d, generator=g) * ch).to(dtype)
        val = torch.randn(t + ring, h, d, generator=g).to(dtype)
        # a constant value group and an all-zero key exercise the clamps
        val[3, 0, :32] = 0.5
        if dtype != torch.float16:   # fp16: 0 + 1e-10 rounds to 0 and the reference divides 0/0
            key[5, h - 1, :] = 0
        query = torch.randn(3, qh, d, generator=g).to(dtype)

        store = CompressedKVStore(d, h, key_bits=kb, value_bits=vb, value_group_size=32,
                                  device=cpu, layer_idx=layer)
        # two chunks, the second ragged, like a prefill followed by a ring flush
        t0 = (t * 2) // 3
        store.append_chunk(key[:t0], val[:t0])
        store.append_chunk(key[t0:t], val[t0:t])
        flat = store.get_flat_cache()
        qz = store.quantizer
        mse = qz.mse_quantizer

        # stage intermediates, recomputed with the reference's own calls
        k_all = key[:t].transpose(0, 1)                     # (H, T, D)
        norms = k_all.norm(dim=-1)
        x_unit = k_all / (norms.unsqueeze(-1) + 1e-10)
        y = rotate_forward(x_unit.float(), mse.Pi)
        mq = mse.quantize(k_all)
        x_hat = mse.dequantize(mq)
        residual = k_all - x_hat
        projected = torch.matmul(residual.float(), qz.S.T)

        recent_k, recent_v = key[t:], val[t:]
        out_hybrid = compute_hybrid_attention(query, store, recent_k, recent_v, qh)
        out_hist = compute_hybrid_attention(query, store, None, None, qh)
        q_hg = query.float().view(3, h, qh // h, d).permute(1, 2, 0, 3).reshape(h, -1, d)
        logits = qz.attention_score(q_hg, flat.prod_q)       # (H, G*3, T), unscaled
        k_deq = qz.dequantize(flat.prod_q)

        vq_single = quantize_values(val[:t].transpose(0, 1), bits=vb, group_size=32)
        assert torch.equal(vq_single.data, flat.value_q.data)

        out = {
            "meta": np.array([d, h, qh, t, ring, kb, vb, layer, seed], np.int64),
            "dtype": np.array(str(dtype).replace("torch.", "")),
            "torch_version": np.array(torch.__version__),
            "centroids": mse.centroids.numpy(),
            "boundaries": mse.boundaries.numpy(),
            "Pi": mse.Pi.numpy(),
            "S": qz.S.numpy(),
            "y": y.numpy(),
            "projected": projected.numpy(),
            "mse_indices": flat.prod_q.mse_indices.numpy(),
            "qjl_signs": flat.prod_q.qjl_signs.numpy(),
            "residual_norms": flat.prod_q.residual_norms.float().numpy(),
            "v_data": flat.value_q.data.numpy(),
            "logits": logits.numpy(),
            "k_dequant": k_deq.float().numpy(),
            "memory_bytes": np.array(store.memory_bytes(), np.int64),
        }
        for key_name, tensor in (("key", key), ("value", val), ("query", query),
                                 ("norms", flat.prod_q.norms), ("x_unit", x_unit),
                                 ("v_scales", flat.value_q.scales), ("v_zeros", flat.value_q.zeros),
                                 ("out_hybrid", out_hybrid), ("out_hist", out_hist)):
            arr, suffix = _np(tensor)
            out[key_name + suffix] = arr
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **out)
        print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB, mem_bytes={store.memory_bytes()}")

    shutil.rmtree(scratch, ignore_errors=True)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python " + os.path.basename(__file__) + " <path to a checkout of the reference (0xSero/turboquant)>")
    main(sys.argv[1])
