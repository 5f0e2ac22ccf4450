"""turboquant_b200: the TurboQuant KV-cache hot path (compress-on-store and
decode attention over compressed K/V) as hand-written sm_100a CUDA behind the
reference's Python API.  Same public names as the reference package
(reference turboquant/__init__.py:1-9)."""

from .codebook import compute_lloyd_max_codebook, get_codebook
from .quantizer import TurboQuantMSE, TurboQuantProd
from .kv_cache import TurboQuantKVCache
from .capture import RingBuffer, KVCaptureEngine
from .store import CompressedKVStore
from .score import compute_hybrid_attention
from .paged_cache import CompressedCacheSpec, CompressedPagedKVCache

__version__ = "0.1.0"
