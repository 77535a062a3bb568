"""Per-batch tensors shared by every layer of a forward pass (rope tables, packing, masks)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch


@dataclass
class PackedSeqParams:
    """Packed ("thd") batch description; field names follow Megatron's ``PackedSeqParams`` so user code
    written for the reference passes the same object (reference ``src/mcore_bridge/model/gpt_model.py:238``)."""
    qkv_format: str = 'thd'
    cu_seqlens_q: Optional[torch.Tensor] = None
    cu_seqlens_kv: Optional[torch.Tensor] = None
    cu_seqlens_q_padded: Optional[torch.Tensor] = None
    cu_seqlens_kv_padded: Optional[torch.Tensor] = None
    max_seqlen_q: Optional[int] = None
    max_seqlen_kv: Optional[int] = None


@dataclass
class ForwardContext:
    cu_seqlens: Optional[torch.Tensor] = None      # int32 [B+1], boundaries in the *full* (pre-CP) token stream
    max_seqlen: Optional[int] = None
    cos: Optional[torch.Tensor] = None             # [T_local_cp, rot/2]
    sin: Optional[torch.Tensor] = None
    position_ids: Optional[torch.Tensor] = None    # [T] positions of the tokens this CP rank holds
    padding_mask: Optional[torch.Tensor] = None    # [T_local] True where the token is padding
    seg_ids: Optional[torch.Tensor] = None         # [T_local] packed-sequence index per token
    seq_start: Optional[torch.Tensor] = None       # [T] int32 first token of each token's sequence (attention kernels)
    num_seqs: Optional[int] = None
    input_ids: Optional[torch.Tensor] = None       # hash-routed MoE layers look at the ids
    extra: Dict[str, Any] = field(default_factory=dict)
    rope_tables: Dict[str, Any] = field(default_factory=dict)  # alternative tables (sliding / compressed / indexer)


def layer_cp_comm_type(config, layer_number: int) -> str:
    """``cp_comm_type`` of one layer (1-based ``layer_number``): a string applies to every layer, a list gives one
    entry per layer (parity: reference ``src/mcore_bridge/model/modules/transformer_layer.py:90-96``)."""
    t = getattr(config, 'cp_comm_type', 'p2p') or 'p2p'
    if isinstance(t, (list, tuple)):
        t = t[min(max(layer_number, 1), len(t)) - 1] if t else 'p2p'
    return str(t)
