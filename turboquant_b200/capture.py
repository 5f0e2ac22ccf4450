"""Write path in front of the store: a ring of exact recent tokens and the
engine that decides when to flush it (reference capture.py:21-240).
"""

from __future__ import annotations

from typing import Optional

import ctypes as C

import torch

from . import _engine as E
from . import _lib
from .store import CompressedKVStore


class RingBuffer:
    """The `capacity` most recent tokens, exact, as (capacity, H, D) key and value tensors.

    Contract of the reference's ring (capture.py:21-131): tokens accumulate until the buffer is full;
    the token that arrives next evicts the WHOLE buffer, and `write` hands back everything that was
    evicted during the call (oldest first), or None.
    """

    def __init__(self, capacity: int, num_kv_heads: int, head_dim: int, device, dtype: torch.dtype = torch.bfloat16):
        if capacity < 1:
            raise ValueError("the ring needs room for at least one token")
        self.capacity, self.num_kv_heads, self.head_dim = capacity, num_kv_heads, head_dim
        self.device, self.dtype = device, dtype
        self._keys = torch.zeros(capacity, num_kv_heads, head_dim, device=device, dtype=dtype)
        self._values = torch.zeros_like(self._keys)
        self._fill = 0                                     # tokens held
        self._seen = 0                                     # tokens ever written
        self._fill_dev: Optional[torch.Tensor] = None      # device mirror of _fill, kept by device_len()
        self._fill_dev_val = -1

    def device_len(self) -> torch.Tensor:
        """(1,) int32 device tensor equal to `size`.  The fused decode step lets the kernel write the new
        token at this position and increment it; the host count follows in `advance_after_device_append`."""
        if self._fill_dev is None:
            self._fill_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._fill_dev_val = 0
        if self._fill_dev_val != self._fill:
            self._fill_dev.fill_(self._fill)
            self._fill_dev_val = self._fill
        return self._fill_dev

    def advance_after_device_append(self) -> None:
        self._fill += 1
        self._fill_dev_val += 1
        self._seen += 1

    @property
    def storage(self):
        """The whole (capacity, H, D) key and value buffers."""
        return self._keys, self._values

    @property
    def size(self) -> int:
        return self._fill

    @property
    def is_full(self) -> bool:
        return self._fill >= self.capacity

    @property
    def total_written(self) -> int:
        return self._seen

    def write(self, key: torch.Tensor, value: torch.Tensor, num_tokens: int):
        """Append `num_tokens` tokens.  Seen as one stream - the tokens held, then the new ones - every
        full buffer's worth that is followed by at least one more token leaves; what stays is the tail of
        1..capacity tokens.  No loop over buffers: the split point is arithmetic."""
        held, cap = self._fill, self.capacity
        total = held + num_tokens
        self._seen += num_tokens
        if num_tokens <= 0:
            return None
        evicted_buffers = (total - 1) // cap               # full buffers with a successor
        cut = evicted_buffers * cap - held                 # new tokens that leave with them
        if evicted_buffers == 0:
            self._keys[held:total] = key[:num_tokens]
            self._values[held:total] = value[:num_tokens]
            self._fill = total
            return None
        out_k = torch.cat((self._keys[:held], key[:cut]), 0)
        out_v = torch.cat((self._values[:held], value[:cut]), 0)
        stay = num_tokens - cut
        self._keys[:stay] = key[cut:num_tokens]
        self._values[:stay] = value[cut:num_tokens]
        self._fill = stay
        return out_k, out_v

    def drain(self):
        """Everything held, as copies; the ring is empty afterwards."""
        if self._fill == 0:
            return None
        taken = self._keys[: self._fill].clone(), self._values[: self._fill].clone()
        self._fill = 0
        return taken

    def peek(self):
        """Views of what is held (None when empty)."""
        if self._fill == 0:
            return None
        return self._keys[: self._fill], self._values[: self._fill]

    def reset(self) -> None:
        self._fill = 0
        self._seen = 0


class KVCaptureEngine:
    """Feeds a CompressedKVStore: prefill goes to the store except the last
    `ring_capacity` tokens, decode tokens go to the ring, a full ring is
    compressed as one chunk when the next token arrives."""

    def __init__(self, store: CompressedKVStore, ring_capacity: int = 128, device=None,
                 dtype: torch.dtype = torch.bfloat16):
        self.store = store
        self.ring = RingBuffer(ring_capacity, store.num_kv_heads, store.head_dim, device or store.device, dtype)
        self._prefill_done = False
        self._host_io = None      # buffers and the argument block of decode_step_host

    @property
    def total_compressed_tokens(self) -> int:
        return self.store.num_tokens

    @property
    def total_buffered_tokens(self) -> int:
        return self.ring.size

    @property
    def total_tokens(self) -> int:
        return self.total_compressed_tokens + self.total_buffered_tokens

    def ingest_prefill(self, key: torch.Tensor, value: torch.Tensor, num_tokens: int) -> None:
        cap = self.ring.capacity
        if num_tokens <= cap:
            self.ring.write(key[:num_tokens], value[:num_tokens], num_tokens)
        else:
            n = num_tokens - cap
            self.store.append_chunk(key[:n], value[:n])
            self.ring.write(key[n:num_tokens], value[n:num_tokens], cap)
        self._prefill_done = True

    def ingest_prefill_from_paged_cache(self, kv_cache_tensor: torch.Tensor, num_tokens: int,
                                        block_table: torch.Tensor, block_size: int) -> None:
        """kv_cache_tensor (2, num_blocks, block_size, H, D); block_table maps logical to physical blocks
        (reference capture.py:187-217).  All but the last `capacity` tokens go from the paged cache into
        the compressed store in one launch that walks the table; only the ring's tokens are gathered."""
        if kv_cache_tensor.shape[2] != block_size:
            raise ValueError(f"block_size {block_size} does not match the cache's {kv_cache_tensor.shape[2]}")
        cap = self.ring.capacity
        n = max(num_tokens - cap, 0)
        self.store.append_from_paged(kv_cache_tensor[0], kv_cache_tensor[1], block_table, n)
        b0, b1 = n // block_size, (num_tokens + block_size - 1) // block_size
        phys = block_table[b0:b1].long()
        lo = n - b0 * block_size
        k = kv_cache_tensor[0].index_select(0, phys).flatten(0, 1)[lo:lo + num_tokens - n]
        v = kv_cache_tensor[1].index_select(0, phys).flatten(0, 1)[lo:lo + num_tokens - n]
        self.ring.write(k, v, num_tokens - n)
        self._prefill_done = True

    def ingest_decode(self, key: torch.Tensor, value: torch.Tensor, num_tokens: int) -> None:
        overflow = self.ring.write(key[:num_tokens], value[:num_tokens], num_tokens)
        if overflow is not None:
            self.store.append_chunk(*overflow)

    def decode_step(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, num_query_heads: int,
                    scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode token in one library call: `ingest_decode(key, value, 1)`
        followed by `compute_hybrid_attention(query, store, *ring.peek(), ...)`
        of the reference (capture.py:205-222, score.py:33-91), with the ring
        write done on the device by the query-preparation launch.

        query (1, Qh, D); key / value (1, H, D) in the ring's dtype -> (1, Qh, D).
        Same results as the two separate calls; no reference counterpart as a
        single call.
        """
        ring, store = self.ring, self.store
        if ring.is_full:                      # the rare step: compress the full ring first
            self.store.append_chunk(*ring.drain())
        E.require_cuda(query, "query")
        if key.dtype != ring.dtype or value.dtype != ring.dtype:
            raise TypeError(f"key/value must be {ring.dtype} like the ring")
        t, qh, d = query.shape
        if t != 1 or qh != num_query_heads or d != store.head_dim:
            raise ValueError(f"decode_step takes one query token of {num_query_heads} x {store.head_dim}")
        rk, rv = ring.storage
        lens = ring.device_len()
        res = E.decode(store.consts, store.pool, store.workspace, query, store.block_table, store.seq_len_device,
                       store.num_tokens, scale=scale, min_history=16, ring_k=rk, ring_v=rv, ring_lens=lens,
                       max_ring_len=ring.size + 1, ring_stride_seq=0, ring_stride_token=rk.stride(0),
                       append_k=key.contiguous(), append_v=value.contiguous(), out=out)
        ring.advance_after_device_append()
        return res

    def decode_step_host(self, host_in: torch.Tensor, host_out: torch.Tensor, num_query_heads: int,
                         scale: Optional[float] = None) -> None:
        """`decode_step` for a caller whose step data lives in host memory.

        host_in: pinned 1-D tensor in the ring's dtype, key (H*D) | value (H*D) | query (Qh*D) of the
        new token; host_out: pinned tensor of Qh*D elements that receives the attention output.
        One library call enqueues the host-to-device copy, the ring append + attention and the
        device-to-host copy on the current stream; nothing is synchronised (synchronise the stream
        before reading host_out).  Same results as `decode_step`.
        """
        ring, store = self.ring, self.store
        if ring.is_full:
            self.store.append_chunk(*ring.drain())
        h, d, qh = store.num_kv_heads, store.head_dim, num_query_heads
        nk, nq = h * d, qh * d
        io = self._host_io
        if io is None or io["qh"] != qh:
            if host_in.dtype != ring.dtype or host_out.dtype != ring.dtype:
                raise TypeError(f"host buffers must be {ring.dtype} like the ring")
            stage = torch.empty(2 * nk + nq, dtype=ring.dtype, device=store.device)
            out = torch.empty(1, qh, d, dtype=ring.dtype, device=store.device)
            rk, rv = ring.storage
            a = _lib.tq_decode_args()
            es = stage.element_size()
            a.append_k, a.append_v = stage.data_ptr(), stage.data_ptr() + nk * es
            a.query, a.q_dtype, a.batch, a.num_q_heads = stage.data_ptr() + 2 * nk * es, E.dtype_code(ring.dtype), 1, qh
            a.ring_k, a.ring_v, a.ring_dtype = rk.data_ptr(), rv.data_ptr(), E.dtype_code(ring.dtype)
            a.ring_stride_seq, a.ring_stride_token, a.ring_capacity = 0, rk.stride(0), ring.capacity
            a.min_history, a.out = 16, out.data_ptr()
            a.scale = scale if scale is not None else 1.0 / (d ** 0.5)
            io = self._host_io = dict(qh=qh, stage=stage, out=out, args=a, argref=C.byref(a),
                                      in_bytes=(2 * nk + nq) * es, out_bytes=nq * es, sms=E.sm_count(store.device))
        if host_in.numel() != 2 * nk + nq or host_out.numel() != nq or not host_in.is_pinned():
            raise ValueError("host_in must be a pinned tensor of key | value | query, host_out of Qh*D elements")
        a = io["args"]
        n, r = store.num_tokens, ring.size + 1
        # everything that depends only on the compressed length, the pool and the ring's 64-token bucket
        plan = (n, (r + 63) >> 6, store.pool.num_blocks, store.workspace.buf.data_ptr())
        if io.get("plan") != plan:
            splits = E.choose_splits(1, h, n, io["sms"], r)
            store.workspace.ensure_decode(store.consts, 1, qh, h, splits)
            plan = plan[:3] + (store.workspace.buf.data_ptr(),)
            a.block_table, a.block_table_stride = store.block_table.data_ptr(), store.block_table.numel()
            a.seq_lens, a.max_seq_len, a.num_splits = store.seq_len_device.data_ptr(), n, splits
            a.workspace, a.workspace_bytes = store.workspace.ptr, store.workspace.nbytes
            a.ring_lens = ring.device_len().data_ptr()
            io["plan"] = plan
            io["consts"], io["pool"] = C.byref(store.consts.c), C.byref(store.pool.c)
            io["stage_ptr"], io["fn"] = io["stage"].data_ptr(), E.lib().tq_decode_host_io
        else:
            ring.device_len()          # keeps the device copy of the ring length in step with host-side writes
        a.max_ring_len = r
        if scale is not None:
            a.scale = scale
        rc = io["fn"](io["consts"], io["pool"], io["argref"], host_in.data_ptr(), io["stage_ptr"], io["in_bytes"],
                      host_out.data_ptr(), io["out_bytes"], torch.cuda.current_stream(store.device).cuda_stream)
        if rc != 0:
            E.check(rc, "tq_decode_host_io")
        ring.advance_after_device_append()

    def flush(self) -> None:
        data = self.ring.drain()
        if data is not None:
            self.store.append_chunk(*data)

    def reset(self) -> None:
        self.ring.reset()
        self.store.reset()
        self._prefill_done = False
