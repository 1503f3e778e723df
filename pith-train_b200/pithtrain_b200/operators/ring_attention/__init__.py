"""Context-parallel ring attention (GQA and MLA), same names as ``pithtrain.operators.ring_attention``."""

from ._ring import (cuda_graphs_enabled, enable_cuda_graphs, enable_peer_copies, peer_copies_enabled,
                    release_cuda_graphs, release_peer_copies)
from .mla import RingMLAAttentionFunc, _online_softmax_combine_log2, ring_mla_attention_func
from .sharding import local_positions, shard_sequence, unshard_sequence
from .standard import RingAttentionFunc, _online_softmax_combine, _ring_send_recv_kv, ring_attention_func

__all__ = [
    "RingAttentionFunc", "RingMLAAttentionFunc", "ring_attention_func", "ring_mla_attention_func",
    "_online_softmax_combine", "_online_softmax_combine_log2", "_ring_send_recv_kv",
    "local_positions", "shard_sequence", "unshard_sequence",
    "enable_cuda_graphs", "cuda_graphs_enabled", "release_cuda_graphs",
    "enable_peer_copies", "peer_copies_enabled", "release_peer_copies",
]
