"""B200 (sm_100a) kernels for the DeepSeek-sparse-attention hot path, behind the entry signatures of
the TileLang-Ascend examples: lightning indexer -> top-k selector -> sparse MLA forward (+ decode,
backward).  Python / PyTorch host code over a C-ABI CUDA library; there is no CPU fallback."""
from . import _lib
from .deepseek_mla import flashattn_mla_decode, mla_decode, mla_decode_tilelang, run_mla_decode
from .hisa import block_sparse_logits_raw, block_sparse_mqa_attn_return_logits, paged_block_sparse_mqa_attn_return_logits
from .host_pipeline import HostPipelinedForward
from .lightning_indexer import indexer, indexer_scores_raw, lightning_indexer, lightning_indexer_raw
from .sharding import (all_reduce_key_gradient, causal_query_costs, shard_batch, shard_queries, shard_range, shard_range_balanced, shard_ranges_by_rounds, block_time_in_rounds, tail_split_plan,
                       sparse_mla_bwd_sharded)
from .sparse_flash_attention import (sparse_attention_fwd, sparse_attn_tilelang, sparse_mla, sparse_mla_bwd_raw,
                                     sparse_mla_fwd_raw)
from .sparse_flash_mla import sink_combine_raw, sparse_flash_mla
from .topk_selector import simple_topk_selector, topk_select_raw

kernel_status = _lib.kernel_status

__all__ = [
    "indexer", "lightning_indexer", "simple_topk_selector", "sparse_attention_fwd", "sparse_attn_tilelang", "mla_decode", "mla_decode_tilelang", "flashattn_mla_decode", "run_mla_decode",
    "sparse_flash_mla", "sink_combine_raw", "block_sparse_mqa_attn_return_logits", "paged_block_sparse_mqa_attn_return_logits", "block_sparse_logits_raw", "sparse_mla", "sparse_mla_fwd_raw", "sparse_mla_bwd_raw", "indexer_scores_raw", "lightning_indexer_raw",
    "topk_select_raw", "HostPipelinedForward", "shard_range", "shard_range_balanced", "shard_ranges_by_rounds", "block_time_in_rounds", "tail_split_plan", "causal_query_costs", "shard_queries", "shard_batch", "all_reduce_key_gradient", "sparse_mla_bwd_sharded", "kernel_status",
]
