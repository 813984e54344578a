"""deserve_b200 — the paged KV-cache hot path of DeServe for NVIDIA B200.

Host classes keep the reference's names (deserve_worker/kvcache/**,
deserve_worker/model/context/flash.py, deserve_worker/task.py); the data
movement and attention run in hand-written sm_100a CUDA kernels behind the C
ABI of libdeserve_kv.so (include/deserve_kv.h).
"""
from .context import FlashDecodeCtx, FlashForwardCtx, FlashPrefillCtx, ForwardCtx, PagedForwardCtx
from .kvcache import (ChunkHandle, ChunkPool, CopiedPinnedMemory, CpuChunkPool, CpuPagePool, GpuPagePool,
                      KVCacheManager, KVConfig, PagedKVCache, PagePool, PageTableAllocator, PageTableHandle,
                      PinnedKVCache, PinnedMemory, VirtualPagedKVCache, VirtualPagePool, check_page_ownership)
from .ops import (BatchDecodeWithPagedKVCacheWrapper, BatchPrefillWithPagedKVCacheWrapper, append_paged_kv_cache,
                  apply_rope, apply_rope_inplace, greedy_sample, paged_decode, paged_prefill, rmsnorm,
                  rope_append_paged_kv_cache, silu_mul)
from .engine import (BatchDecode, BatchPrefill, BatchResult, KVStage, MicroBatchProcessor, RingPipeline, StageProcessor,
                     StepRequest, make_ring_links)
from .model import LlamaStage, ModelArgs
from .task import SamplingParams, TaskData, TaskManager
from .request import InitRequest
from .scheduling import DecodeFirstJoin, PrefillFirstJoin, StepPlanner, SwapPolicy, VanillaJoin
from . import wire

__all__ = [n for n in dir() if not n.startswith("_")]
