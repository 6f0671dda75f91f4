"""B200-native (sm_100a) KV-cache, RoPE and chunked grouped-query attention behind the call
surface of the Strata / ``ollm`` runtime.  Importing the package needs the built C-ABI library
(``python lokahi_b200/build.py``); there is no CPU or PyTorch fallback for any compute call."""
from ._lib import DeviceFlagError, NotResidentError, OutOfPagesError
from .attention import PagedView, check_dense_attention_status, chunked_grouped_attention, chunked_grouped_attention_no_mask
from .backend import B200Backend, BackendError, register
from .batching import BatchedDecodeLoop, DecodeRequest
from .decoder import PagedDecoder
from .generation import greedy_generate
from .hostpipe import HostStepPipeline
from .tracing import TensorTracer, TraceEvent
from .glue import add_rms_norm, rms_norm, swiglu
from .kvcache import PagedKVCache, PagedLlamaDiskCache, PagedQwen3NextDiskCache, create_paged_kv_cache
from .residency import BudgetExceededError, GroupState, KVPageResidency
from .prefetch import KVPageLease, KVPagePrefetcher, KVPrefetchSnapshot
from .sharding import HeadShard, InterleavedShard, PeerExchange, PeerGather, PeerSeqMerge, SequenceShard, gather_head_outputs, sequence_sharded_decode
from .pool import PagedKVConfig, PagedPool, merge_partials, rope_inv_freq, rope_rows

register()

__all__ = [
    "B200Backend", "BatchedDecodeLoop", "HostStepPipeline", "DecodeRequest", "BudgetExceededError", "InterleavedShard", "PeerExchange", "PeerSeqMerge", "check_dense_attention_status", "TensorTracer", "TraceEvent", "add_rms_norm", "rms_norm", "swiglu", "GroupState", "KVPageLease", "KVPagePrefetcher", "KVPrefetchSnapshot", "KVPageResidency", "HeadShard", "PeerGather", "SequenceShard", "gather_head_outputs", "merge_partials", "sequence_sharded_decode", "BackendError", "DeviceFlagError", "NotResidentError", "OutOfPagesError", "PagedKVCache", "PagedQwen3NextDiskCache",
    "PagedDecoder", "PagedKVConfig", "PagedLlamaDiskCache", "PagedPool", "PagedView", "chunked_grouped_attention",
    "chunked_grouped_attention_no_mask", "create_paged_kv_cache", "greedy_generate", "register",
    "rope_inv_freq", "rope_rows",
]
