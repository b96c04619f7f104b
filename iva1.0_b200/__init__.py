"""B200-native paged-KV decode path behind the reference's operator signatures.

Three operators, each a hand-written sm_100a CUDA kernel reached through a C-ABI
shared library (``libivab.so``, declared in ``include/ivab.h``):

* KV append  -- ``kv_ops(cache, indices, values, "scatter")`` / ``paged_append``
* KV gather  -- ``kv_ops(cache, indices, operation="gather")`` / ``paged_gather``
* single-query decode attention through a block table -- ``paged_decode_attention``,
  ``attention(q, k, v, scale)`` and the ``AttentionB200`` module.

There is no CPU or PyTorch fallback: every operator raises if the library is missing
or the tensors are not on a CUDA device.
"""

from . import workloads  # noqa: F401
from ._lib import IvabError, lib_path, load_library  # noqa: F401
from .kv_ops import kv_ops, kv_compact, paged_append, paged_gather  # noqa: F401
from .attention import (  # noqa: F401
    AttentionB200,
    attention,
    decode_workspace_bytes,
    get_attention,
    paged_decode_attention,
    paged_decode_step,
)
from .paged_cache import PagedKVCache  # noqa: F401
from .decode_step import GraphedDecodeStep  # noqa: F401
from .decode_loop import decode_loop  # noqa: F401
from .sharding import HeadParallelDecoder, shard_requests  # noqa: F401

__version__ = "0.1.0"
