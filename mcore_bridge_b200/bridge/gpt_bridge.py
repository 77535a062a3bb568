"""``GPTBridge``: Hugging Face safetensors <-> the sharded model, in both directions, streaming layer by layer.

Public surface (parity: reference ``src/mcore_bridge/bridge/gpt_bridge.py:1888-2022``):
``load_weights(mg_models, hf_model_dir, peft_format, adapter_name, converter)``,
``export_weights(...)`` (a generator of ``(hf_name, tensor)``) and ``save_weights(...)``.

Design.  Every tensor of the model is described once by a *slot*: where it lives in the model, which
Hugging Face keys it corresponds to, how it is sharded (``tp_dim``: 0 = rows, 1 = columns, ``'glu'`` = the
``[gate; up]`` stacking whose halves are sharded separately, ``None`` = replicated) and an optional pair of
pure functions that re-lay the *full* tensor (QKV interleaving per query group, gate/up stacking, expert
stacking, vocabulary padding ...).  One walker drives all slots in a fixed global order; the direction flag
only selects which half of each slot runs:

* load: every rank reads the tensors it needs from disk, applies the re-layout, takes its shard. No
  communication.
* export: every rank walks the same slots in lock-step; shards are all-gathered over the tensor-parallel
  (or expert-tensor-parallel) group, local experts over the expert-parallel group, and layers owned by
  another pipeline stage are broadcast from their owner, so any rank (by default only the master) can
  write the file.

The module works on CPU tensors with gloo as well as on GPUs with NCCL: control tensors are created on the
device of the parameters.
"""
from __future__ import annotations

import re
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..parallel import state as ps
from ..utils.dequantizer import Fp8Dequantizer, add_dequantized_views
from ..utils.env import is_master
from ..utils.logger import get_logger
from ..utils.safetensors import LazyTensor, SafetensorLazyLoader, StreamingSafetensorSaver
from ..utils.utils import deep_getattr

logger = get_logger()

_DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float8_e4m3fn: 3, torch.int64: 4,
                torch.int32: 5, torch.uint8: 6, torch.bool: 7, torch.float64: 8}
_CODE_DTYPES = {v: k for k, v in _DTYPE_CODES.items()}


# ---------------------------------------------------------------------------------------------------------
# pure re-layout helpers (full tensors, no parallelism)
# ---------------------------------------------------------------------------------------------------------
def qkv_to_mcore(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_query_groups: int) -> torch.Tensor:
    """``[q; k; v]`` (HF, head-major) -> per-query-group interleaving ``[g0: q.. k v | g1: q.. k v | ...]``."""
    tail = q.shape[1:]
    g = num_query_groups
    parts = [t.reshape(g, -1, *tail) for t in (q, k, v)]
    return torch.cat(parts, dim=1).reshape(-1, *tail)


def qkv_to_hf(qkv: torch.Tensor, num_query_groups: int, q_rows_per_group: int, kv_rows_per_group: int):
    tail = qkv.shape[1:]
    x = qkv.reshape(num_query_groups, q_rows_per_group + 2 * kv_rows_per_group, *tail)
    q = x[:, :q_rows_per_group].reshape(-1, *tail)
    k = x[:, q_rows_per_group:q_rows_per_group + kv_rows_per_group].reshape(-1, *tail)
    v = x[:, q_rows_per_group + kv_rows_per_group:].reshape(-1, *tail)
    return q, k, v


def shard(full: torch.Tensor, tp_dim, rank: int, size: int) -> torch.Tensor:
    if size == 1 or tp_dim is None:
        return full
    if tp_dim == 'glu':
        x = full.reshape(2, full.shape[0] // 2, *full.shape[1:])
        return x.chunk(size, dim=1)[rank].reshape(-1, *full.shape[1:])
    return full.chunk(size, dim=tp_dim)[rank]


def unshard(parts: List[torch.Tensor], tp_dim) -> torch.Tensor:
    if len(parts) == 1 or tp_dim is None:
        return parts[0]
    if tp_dim == 'glu':
        xs = [p.reshape(2, p.shape[0] // 2, *p.shape[1:]) for p in parts]
        return torch.cat(xs, dim=1).reshape(-1, *parts[0].shape[1:])
    return torch.cat(parts, dim=tp_dim)


def gdn_in_proj_to_hf(full: torch.Tensor, cfg, split: bool) -> Dict[str, torch.Tensor]:
    """Rows of the fused gated-DeltaNet input projection (per key-head group ``[q | k | v | z | b | a]``) -> the
    Hugging Face tensors: ``in_proj_qkvz`` / ``in_proj_ba`` (grouped per key head), or with ``split`` the four flat
    ``in_proj_qkv`` (``[all q | all k | all v]``) / ``in_proj_z`` / ``in_proj_b`` / ``in_proj_a``.  Only dim 0 is
    re-laid, so the same mapping serves the weight ``[out, H]`` and a LoRA ``lora_B`` ``[out, r]``."""
    nk, nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    ratio = nv // nk
    gq, gba = 2 * dk + 2 * ratio * dv, 2 * ratio
    tail = full.shape[1:]
    g = full.reshape(nk, gq + gba, *tail)
    if not split:
        return {'in_proj_qkvz': g[:, :gq].reshape(-1, *tail), 'in_proj_ba': g[:, gq:].reshape(-1, *tail)}
    q, k, v = g[:, :dk], g[:, dk:2 * dk], g[:, 2 * dk:2 * dk + ratio * dv]
    return {'in_proj_qkv': torch.cat([q.reshape(-1, *tail), k.reshape(-1, *tail), v.reshape(-1, *tail)], 0),
            'in_proj_z': g[:, 2 * dk + ratio * dv:gq].reshape(-1, *tail),
            'in_proj_b': g[:, gq:gq + ratio].reshape(-1, *tail),
            'in_proj_a': g[:, gq + ratio:].reshape(-1, *tail)}


def gdn_in_proj_to_mcore(parts: Dict[str, torch.Tensor], cfg, split: bool) -> torch.Tensor:
    """Inverse of :func:`gdn_in_proj_to_hf`."""
    nk, nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    ratio = nv // nk
    gq, gba = 2 * dk + 2 * ratio * dv, 2 * ratio
    if not split:
        qkvz, ba = parts['in_proj_qkvz'], parts['in_proj_ba']
        tail = qkvz.shape[1:]
        return torch.cat([qkvz.reshape(nk, gq, *tail), ba.reshape(nk, gba, *tail)], dim=1).reshape(-1, *tail)
    qkv = parts['in_proj_qkv']
    tail = qkv.shape[1:]
    pieces = [qkv[:nk * dk].reshape(nk, dk, *tail), qkv[nk * dk:2 * nk * dk].reshape(nk, dk, *tail),
              qkv[2 * nk * dk:].reshape(nk, ratio * dv, *tail), parts['in_proj_z'].reshape(nk, ratio * dv, *tail),
              parts['in_proj_b'].reshape(nk, ratio, *tail), parts['in_proj_a'].reshape(nk, ratio, *tail)]
    return torch.cat(pieces, dim=1).reshape(-1, *tail)


class GPTBridge:
    # ---- Hugging Face naming; families override what differs
    hf_layers_prefix = 'model.layers'
    hf_embed_key = 'model.embed_tokens.weight'
    hf_final_layernorm_key = 'model.norm.weight'
    hf_lm_head_key = 'lm_head.weight'
    hf_score_key = 'score.weight'
    # published checkpoint key prefixes -> the in-memory layout (applied to the key index on load, inverted on export)
    hf_state_dict_mapping: Dict[str, str] = {}
    hf_load_aliases: Dict[str, str] = {}     # further prefixes accepted on load only (older published layouts)
    split_gdn_projections = False            # gated-DeltaNet input projection stored as qkv / z / b / a tensors
    hf_attn_prefix = 'self_attn'
    hf_mlp_prefix = 'mlp'
    hf_q_norm_key = 'q_norm.weight'
    hf_k_norm_key = 'k_norm.weight'
    hf_o_proj_key = 'o_proj.weight'
    hf_input_layernorm_key = 'input_layernorm.weight'
    hf_post_attention_layernorm_key = 'post_attention_layernorm.weight'
    hf_gate_key = 'gate.weight'
    hf_expert_bias_key = 'gate.e_score_correction_bias'
    hf_expert_bias_2d = False                # stored as ``[1, E]`` (Ernie-4.5)
    hf_shared_expert_prefix = None           # resolved per family ('shared_expert' / 'shared_experts')
    hf_shared_expert_gate_key = 'shared_expert_gate.weight'
    hf_experts_prefix = 'experts'
    hf_expert_proj_names = ('gate_proj', 'up_proj', 'down_proj')     # per-expert linear names (MiniMax: w1 / w3 / w2)
    hf_fused_gate_up = False                 # dense MLP exported as one ``gate_up_proj`` tensor (GLM-4)
    # routed experts exported as ``experts.gate_up_proj`` / ``experts.down_proj``
    hf_fused_experts = False
    # layout written for fused expert tensors when no checkpoint was loaded: input-major ``[E, H, 2F]`` / ``[E, F, H]``
    hf_experts_transposed = False
    hf_fused_qkv_key = None                  # e.g. 'query_key_value': one tensor laid out [all q | all k | all v]
    fp8_block_size = 128

    def __init__(self, config):
        self.config = config
        self._peft_format = False
        self._adapter_name = 'default'
        self._target_device = None
        self._only_master_rank = False
        self._fp8_dequant = Fp8Dequantizer((self.fp8_block_size, self.fp8_block_size))
        self.export_fp8 = False
        llm = config.llm_model_type or config.hf_model_type or ''
        if self.hf_shared_expert_prefix is None:
            self.hf_shared_expert_prefix = 'shared_expert' if llm.startswith('qwen') else 'shared_experts'

    # ------------------------------------------------------------------ parallel helpers
    @property
    def tp_size(self):
        return ps.get_world_size('tp')

    @property
    def tp_rank(self):
        return ps.get_rank_in('tp') if self.tp_size > 1 else 0

    def _group_info(self, is_expert: bool):
        name = 'etp' if is_expert else 'tp'
        n = ps.get_world_size(name)
        return name, n, (ps.get_rank_in(name) if n > 1 else 0)

    def _all_gather_tp(self, local: Optional[torch.Tensor], tp_dim, is_expert: bool) -> Optional[torch.Tensor]:
        name, n, _ = self._group_info(is_expert)
        if local is None or n == 1 or tp_dim is None:
            return local
        parts = [torch.empty_like(local) for _ in range(n)]
        dist.all_gather(parts, local.contiguous(), group=ps.get_group(name))
        return unshard(parts, tp_dim)

    def _all_gather_ep(self, local: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """``[E_local, ...]`` on every EP rank -> ``[E, ...]``."""
        n = ps.get_world_size('ep')
        if local is None or n == 1:
            return local
        out = torch.empty((n * local.shape[0], *local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=ps.get_group('ep'))
        return out

    def _broadcast_pp(self, tensor: Optional[torch.Tensor], device) -> Optional[torch.Tensor]:
        """Every pipeline rank gets the tensor held by the one stage that owns it (owner found by all-reduce)."""
        n = ps.get_world_size('pp')
        if n == 1:
            return tensor
        group = ps.get_group('pp')
        me = dist.get_rank()
        flag = torch.tensor([me if tensor is not None else -1], dtype=torch.int64, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        src = int(flag.item())
        if src < 0:
            return None
        meta = torch.zeros(10, dtype=torch.int64, device=device)
        if tensor is not None and me == src:
            meta[0] = tensor.dim()
            meta[1] = _DTYPE_CODES[tensor.dtype]
            for i, s in enumerate(tensor.shape):
                meta[2 + i] = s
        dist.broadcast(meta, src=src, group=group)
        if me != src:
            m = meta.tolist()
            tensor = torch.empty(m[2:2 + m[0]], dtype=_CODE_DTYPES[m[1]], device=device)
        else:
            tensor = tensor.contiguous()
        dist.broadcast(tensor, src=src, group=group)
        return tensor

    def _agree(self, value: bool, device) -> bool:
        """Logical OR of a flag over the pipeline group, so ranks without the layer follow the owner's branch."""
        if ps.get_world_size('pp') == 1:
            return value
        t = torch.tensor([int(bool(value))], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ps.get_group('pp'))
        return bool(t.item())

    @property
    def _device(self):
        if torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == 'nccl':
            return torch.device('cuda', torch.cuda.current_device())
        return torch.device('cpu')

    # ------------------------------------------------------------------ slot primitives
    def _load_hf(self, hf_sd: Dict[str, LazyTensor], key: str) -> torch.Tensor:
        t = hf_sd[key].load()
        sk = key + '_scale_inv'
        if sk in hf_sd and t.dtype in (torch.float8_e4m3fn, torch.uint8):
            t = self._fp8_dequant.convert(t, hf_sd[sk].load())
        return t

    def _put(self, param: Optional[torch.Tensor], full: torch.Tensor, tp_dim, is_expert: bool = False):
        """Copy this rank's shard of ``full`` into ``param``."""
        if param is None:
            return
        _, n, r = self._group_info(is_expert)
        src = shard(full, tp_dim, r, n)
        if tuple(src.shape) != tuple(param.shape):
            raise ValueError(f'shape mismatch: checkpoint shard {tuple(src.shape)} vs parameter {tuple(param.shape)}')
        with torch.no_grad():
            param.copy_(src.to(device=param.device, dtype=param.dtype))

    def _get(self, param: Optional[torch.Tensor], tp_dim, is_expert: bool = False, ep_gather: bool = False
             ) -> Optional[torch.Tensor]:
        """Full tensor assembled from all shards; identical on every rank of the model-parallel group."""
        t = None if param is None else param.detach()
        t = self._all_gather_tp(t, tp_dim, is_expert)
        if ep_gather:
            t = self._all_gather_ep(t)
        t = self._broadcast_pp(t, self._device)
        return t

    def _emit(self, out: Dict[str, torch.Tensor], key: str, tensor: Optional[torch.Tensor]):
        if tensor is None:
            return
        if self._only_master_rank and not is_master():
            return
        t = tensor.to(self._target_device) if self._target_device is not None else tensor
        if t.data_ptr() == tensor.data_ptr():
            t = t.clone()  # never hand out a view of a live parameter
        out[key] = t

    def _direct(self, module, attr: str, hf_sd, hf_key: str, to_mcore: bool, tp_dim=None, is_expert=False,
                optional: bool = False, to_mg: Optional[Callable] = None, to_hf: Optional[Callable] = None):
        """One tensor <-> one key.  ``to_mg`` / ``to_hf`` re-lay the full tensor."""
        param = deep_getattr(module, attr) if module is not None else None
        if to_mcore:
            if param is None:
                return
            if hf_key not in hf_sd:
                if optional:
                    return
                raise KeyError(f'{hf_key} is missing from the checkpoint')
            full = self._load_hf(hf_sd, hf_key)
            if to_mg is not None:
                full = to_mg(full)
            self._put(param, full, tp_dim, is_expert)
        else:
            exists = self._agree(param is not None, self._device)
            if not exists:
                return
            full = self._get(param, tp_dim, is_expert)
            if full is not None and to_hf is not None:
                full = to_hf(full)
            self._emit(hf_sd, hf_key, full)

    # ------------------------------------------------------------------ embeddings / head
    def _pad_vocab(self, w: torch.Tensor, rows: int) -> torch.Tensor:
        if w.shape[0] == rows:
            return w
        if w.shape[0] > rows:
            return w[:rows]
        pad = torch.zeros((rows - w.shape[0], *w.shape[1:]), dtype=w.dtype)
        return torch.cat([w, pad], dim=0)

    def _vocab_rows(self) -> int:
        from ..models.gpt_model import padded_vocab
        return padded_vocab(self.config.padded_vocab_size, self.tp_size)

    def _convert_pre_process(self, model, hf_sd, to_mcore: bool):
        has = model is not None and getattr(model, 'pre_process', False) and model.embedding is not None
        rows, actual = self._vocab_rows(), self.config.padded_vocab_size
        self._direct(model.embedding.word_embeddings if has else None, 'weight', hf_sd, self.hf_embed_key, to_mcore,
                     tp_dim=0, to_mg=lambda w: self._pad_vocab(w, rows), to_hf=lambda w: w[:actual])

    def _convert_post_process(self, model, hf_sd, to_mcore: bool):
        cfg = self.config
        has = model is not None and getattr(model, 'post_process', False)
        dec = model.decoder if has else None
        self._direct(dec, 'final_layernorm.weight', hf_sd, self.hf_final_layernorm_key, to_mcore)
        if cfg.enable_hyper_connections:
            head_prefix = self.hf_final_layernorm_key.rsplit('norm.weight', 1)[0]
            self._set_hyper_connection(dec.hc_head if has else None, hf_sd, head_prefix, 'head', to_mcore)
        if cfg.task_type == 'seq_cls':
            self._direct(model if has else None, 'output_layer.weight', hf_sd, self.hf_score_key, to_mcore)
            return
        if cfg.task_type == 'embedding':
            return
        if not cfg.untie_embeddings_and_output_weights:
            # tied: the head shares the embedding matrix; a last pipeline stage with its own copy loads it too
            if to_mcore and has and not getattr(model, 'pre_process', False):
                rows = self._vocab_rows()
                self._direct(model, 'output_layer.weight', hf_sd, self.hf_embed_key, True, tp_dim=0,
                             to_mg=lambda w: self._pad_vocab(w, rows))
            return
        rows, actual = self._vocab_rows(), cfg.padded_vocab_size
        self._direct(model if has else None, 'output_layer.weight', hf_sd, self.hf_lm_head_key, to_mcore, tp_dim=0,
                     to_mg=lambda w: self._pad_vocab(w, rows), to_hf=lambda w: w[:actual])

    # ------------------------------------------------------------------ attention
    def _set_qkv(self, attn, hf_sd, prefix: str, to_mcore: bool):
        cfg = self.config
        ng = cfg.num_query_groups
        d = cfg.kv_channels
        q_rows = d * cfg.num_attention_heads // ng * (2 if cfg.attention_output_gate else 1)
        names = ['q_proj', 'k_proj', 'v_proj']
        for suffix, attr in (('weight', 'linear_qkv.weight'), ('bias', 'linear_qkv.bias')):
            param = deep_getattr(attn, attr) if attn is not None else None
            if to_mcore:
                if param is None:
                    continue
                if self.hf_fused_qkv_key is not None:
                    fk = f'{prefix}{self.hf_fused_qkv_key}.{suffix}'
                    if suffix == 'bias' and fk not in hf_sd:
                        continue
                    w = self._load_hf(hf_sd, fk)
                    nq_rows, kv_rows = q_rows * ng, d * ng
                    parts = [w[:nq_rows], w[nq_rows:nq_rows + kv_rows], w[nq_rows + kv_rows:]]
                else:
                    keys = [f'{prefix}{n}.{suffix}' for n in names]
                    if suffix == 'bias' and keys[0] not in hf_sd:
                        continue
                    parts = [self._load_hf(hf_sd, k) for k in keys]
                full = qkv_to_mcore(*parts, ng)
                self._put(param, full, 0)
            else:
                if not self._agree(param is not None, self._device):
                    continue
                full = self._get(param, 0)
                if full is None:
                    continue
                if self.hf_fused_qkv_key is not None:
                    self._emit(hf_sd, f'{prefix}{self.hf_fused_qkv_key}.{suffix}',
                               torch.cat(list(qkv_to_hf(full, ng, q_rows, d)), dim=0))
                    continue
                for n, t in zip(names, qkv_to_hf(full, ng, q_rows, d)):
                    self._emit(hf_sd, f'{prefix}{n}.{suffix}', t)

    def _set_layer_attn(self, layer, hf_sd, prefix: str, to_mcore: bool):
        cfg = self.config
        attn = layer.self_attention if layer is not None else None
        ap = f'{prefix}{self.hf_attn_prefix}.'
        if self._layer_is_linear_attention(prefix, 'lightning'):
            self._set_lightning(layer, attn, hf_sd, prefix, ap, to_mcore)
            return
        if cfg.multi_latent_attention:
            self._set_mla(layer, attn, hf_sd, prefix, ap, to_mcore)
            return
        if self._layer_is_linear_attention(prefix):
            self._set_gdn(attn, hf_sd, prefix, to_mcore)
            return
        self._set_qkv(attn, hf_sd, ap, to_mcore)
        self._direct(attn, 'linear_proj.weight', hf_sd, ap + self.hf_o_proj_key, to_mcore, tp_dim=1)
        self._direct(attn, 'linear_proj.bias', hf_sd, ap + self.hf_o_proj_key.replace('weight', 'bias'), to_mcore,
                     optional=True)
        if cfg.qk_layernorm and cfg.qk_layernorm_full:
            self._direct(attn, 'q_norm.weight', hf_sd, ap + self.hf_q_norm_key, to_mcore, tp_dim=0)
            self._direct(attn, 'k_norm.weight', hf_sd, ap + self.hf_k_norm_key, to_mcore, tp_dim=0)
        elif cfg.qk_layernorm:
            self._direct(attn, 'q_layernorm.weight', hf_sd, ap + self.hf_q_norm_key, to_mcore)
            self._direct(attn, 'k_layernorm.weight', hf_sd, ap + self.hf_k_norm_key, to_mcore)
        if cfg.post_sublayer_layernorm:
            self._direct(attn, 'post_self_attn_layernorm.weight', hf_sd, prefix + 'post_self_attn_layernorm.weight',
                         to_mcore)
            self._direct(layer.mlp if layer is not None else None, 'post_mlp_layernorm.weight', hf_sd,
                         prefix + 'post_mlp_layernorm.weight', to_mcore)
        if cfg.softmax_type == 'learnable':
            self._direct(attn, 'core_attention.softmax_offset', hf_sd, ap + 'sinks', to_mcore, tp_dim=0)
        self._direct(attn, 'linear_qkv.layer_norm_weight', hf_sd, prefix + self.hf_input_layernorm_key, to_mcore)

    hf_linear_attn_prefix = 'linear_attn'

    def _set_lightning(self, layer, attn, hf_sd, prefix: str, ap: str, to_mcore: bool):
        """Lightning-attention layers of the Ling / Ring hybrids: ordinary fused QKV, per-head q/k norms, the output
        gate projection ``g_proj`` (column parallel) and the group norm ``g_norm`` (sharded with the heads)
        (reference ``src/mcore_bridge/model/gpts/bailing_hybrid.py:27-45``)."""
        cfg = self.config
        self._direct(layer, 'input_layernorm.weight', hf_sd, prefix + self.hf_input_layernorm_key, to_mcore)
        self._set_qkv(attn, hf_sd, ap, to_mcore)
        self._direct(attn, 'linear_proj.weight', hf_sd, ap + self.hf_o_proj_key, to_mcore, tp_dim=1)
        if cfg.qk_layernorm:
            self._direct(attn, 'q_layernorm.weight', hf_sd, ap + self.hf_q_norm_key, to_mcore)
            self._direct(attn, 'k_layernorm.weight', hf_sd, ap + self.hf_k_norm_key, to_mcore)
        self._direct(attn, 'g_proj.weight', hf_sd, ap + 'g_proj.weight', to_mcore, tp_dim=0)
        self._direct(attn, 'g_norm.weight', hf_sd, ap + 'g_norm.weight', to_mcore, tp_dim=0)

    def _layer_is_linear_attention(self, prefix: str, variant: str = 'gated_delta_net') -> bool:
        cfg = self.config
        if cfg.linear_attention_freq is None or cfg.experimental_attention_variant != variant:
            return False
        m = re.search(r'\.(\d+)\.$', prefix)
        idx = int(m.group(1)) if m else 0
        pat = cfg.linear_attention_pattern()
        return idx < len(pat) and bool(pat[idx])

    def _set_gdn(self, attn, hf_sd, prefix: str, to_mcore: bool):
        """Gated DeltaNet.  HF keeps ``in_proj_qkvz`` / ``in_proj_ba`` (each grouped per key head) and a conv whose
        channels run ``[all q | all k | all v]``; the model fuses the two projections per key-head group and orders
        the conv channels per group ``[q | k | v]`` so tensor parallelism can shard whole groups."""
        cfg = self.config
        nk, nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        ratio = nv // nk
        gq, gba = 2 * dk + 2 * ratio * dv, 2 * ratio
        lp = f'{prefix}{self.hf_linear_attn_prefix}.'

        def conv_to_mg(w):      # [C, 1, K]: [Q | K | V] -> per group [q | k | v]
            q, k, v = w[:nk * dk], w[nk * dk:2 * nk * dk], w[2 * nk * dk:]
            tail = w.shape[1:]
            return torch.cat([q.reshape(nk, dk, *tail), k.reshape(nk, dk, *tail), v.reshape(nk, ratio * dv, *tail)],
                             dim=1).reshape(-1, *tail)

        def conv_to_hf(w):
            tail = w.shape[1:]
            g = w.reshape(nk, 2 * dk + ratio * dv, *tail)
            return torch.cat([g[:, :dk].reshape(-1, *tail), g[:, dk:2 * dk].reshape(-1, *tail),
                              g[:, 2 * dk:].reshape(-1, *tail)], dim=0)

        param = attn.in_proj.weight if attn is not None else None
        split = self.split_gdn_projections
        names = ('in_proj_qkv', 'in_proj_z', 'in_proj_b', 'in_proj_a') if split else ('in_proj_qkvz', 'in_proj_ba')
        if to_mcore:
            if param is not None:
                parts = {n: self._load_hf(hf_sd, f'{lp}{n}.weight') for n in names}
                self._put(param, gdn_in_proj_to_mcore(parts, cfg, split), 0)
        elif self._agree(param is not None, self._device):
            full = self._get(param, 0)
            if full is not None:
                for n, t in gdn_in_proj_to_hf(full, cfg, split).items():
                    self._emit(hf_sd, f'{lp}{n}.weight', t)
        self._direct(attn, 'conv1d.weight', hf_sd, lp + 'conv1d.weight', to_mcore, tp_dim=0, to_mg=conv_to_mg,
                     to_hf=conv_to_hf)
        self._direct(attn, 'A_log', hf_sd, lp + 'A_log', to_mcore, tp_dim=0)
        self._direct(attn, 'dt_bias', hf_sd, lp + 'dt_bias', to_mcore, tp_dim=0)
        self._direct(attn, 'out_norm.weight', hf_sd, lp + 'norm.weight', to_mcore)
        self._direct(attn, 'out_proj.weight', hf_sd, lp + 'out_proj.weight', to_mcore, tp_dim=1)
        self._direct(attn, 'in_proj.layer_norm_weight', hf_sd, prefix + self.hf_input_layernorm_key, to_mcore)

    def _set_mla(self, layer, attn, hf_sd, prefix, ap, to_mcore):
        cfg = self.config
        self._direct(layer, 'input_layernorm.weight', hf_sd, prefix + self.hf_input_layernorm_key, to_mcore)
        if cfg.q_lora_rank is None:
            self._direct(attn, 'linear_q_proj.weight', hf_sd, ap + 'q_proj.weight', to_mcore, tp_dim=0)
        else:
            self._direct(attn, 'linear_q_down_proj.weight', hf_sd, ap + 'q_a_proj.weight', to_mcore)
            self._direct(attn, 'linear_q_up_proj.layer_norm_weight', hf_sd, ap + 'q_a_layernorm.weight', to_mcore)
            self._direct(attn, 'linear_q_up_proj.weight', hf_sd, ap + 'q_b_proj.weight', to_mcore, tp_dim=0)
        self._direct(attn, 'linear_kv_down_proj.weight', hf_sd, ap + 'kv_a_proj_with_mqa.weight', to_mcore)
        self._direct(attn, 'linear_kv_up_proj.layer_norm_weight', hf_sd, ap + 'kv_a_layernorm.weight', to_mcore)
        self._direct(attn, 'linear_kv_up_proj.weight', hf_sd, ap + 'kv_b_proj.weight', to_mcore, tp_dim=0)
        self._direct(attn, 'linear_proj.weight', hf_sd, ap + 'o_proj.weight', to_mcore, tp_dim=1)
        if cfg.experimental_attention_variant == 'dsa':
            ip = ap + 'indexer.'
            idx = attn.indexer if attn is not None else None
            self._direct(idx, 'linear_wq_b.weight', hf_sd, ip + 'wq_b.weight', to_mcore)
            self._direct(idx, 'linear_wk.weight', hf_sd, ip + 'wk.weight', to_mcore)
            self._direct(idx, 'k_norm.weight', hf_sd, ip + 'k_norm.weight', to_mcore)
            self._direct(idx, 'k_norm.bias', hf_sd, ip + 'k_norm.bias', to_mcore, optional=True)
            self._direct(idx, 'linear_weights_proj.weight', hf_sd, ip + 'weights_proj.weight', to_mcore)

    # ------------------------------------------------------------------ MLP / MoE
    def _set_glu(self, fc1_module, attr: str, hf_sd, prefix: str, to_mcore: bool, is_expert: bool = False,
                 gate_name='gate_proj', up_name='up_proj'):
        """``gate_proj`` / ``up_proj`` <-> stacked ``[gate; up]`` (or a fused ``gate_up_proj`` key)."""
        for suffix in ('weight', 'bias'):
            sattr = attr if suffix == 'weight' else attr[:-len('weight')] + 'bias'
            p = deep_getattr(fc1_module, sattr) if fc1_module is not None else None
            gk, uk = f'{prefix}{gate_name}.{suffix}', f'{prefix}{up_name}.{suffix}'
            fused = f'{prefix}gate_up_proj.{suffix}'
            tp_dim = 'glu' if self.config.gated_linear_unit else 0
            if to_mcore:
                if p is None:
                    continue
                if gk in hf_sd:
                    full = torch.cat([self._load_hf(hf_sd, gk), self._load_hf(hf_sd, uk)], dim=0)
                elif fused in hf_sd:
                    full = self._load_hf(hf_sd, fused)
                elif suffix == 'bias':
                    continue
                else:
                    raise KeyError(f'{gk} is missing from the checkpoint')
                self._put(p, full, tp_dim, is_expert)
            else:
                if not self._agree(p is not None, self._device):
                    continue
                full = self._get(p, tp_dim, is_expert)
                if full is None:
                    continue
                if self.hf_fused_gate_up:
                    self._emit(hf_sd, fused, full)
                    continue
                g, u = full.chunk(2, dim=0)
                self._emit(hf_sd, gk, g)
                self._emit(hf_sd, uk, u)

    def _set_dense_mlp(self, mlp, hf_sd, prefix: str, to_mcore: bool, is_expert: bool = False):
        cfg = self.config
        if cfg.gated_linear_unit:
            self._set_glu(mlp, 'linear_fc1.weight', hf_sd, prefix, to_mcore, is_expert)
        else:
            self._direct(mlp, 'linear_fc1.weight', hf_sd, prefix + 'up_proj.weight', to_mcore, tp_dim=0)
            self._direct(mlp, 'linear_fc1.bias', hf_sd, prefix + 'up_proj.bias', to_mcore, tp_dim=0, optional=True)
        self._direct(mlp, 'linear_fc2.weight', hf_sd, prefix + 'down_proj.weight', to_mcore, tp_dim=1,
                     is_expert=is_expert)
        self._direct(mlp, 'linear_fc2.bias', hf_sd, prefix + 'down_proj.bias', to_mcore, optional=True)

    def _set_experts(self, experts, hf_sd, prefix: str, to_mcore: bool):
        """Routed experts.  HF side is either per-expert keys (``experts.{e}.gate_proj.weight`` ...) or fused
        tensors (``experts.gate_up_proj`` ``[E, 2F, H]`` / ``experts.down_proj`` ``[E, H, F]``).  Model side is one
        stacked tensor per linear holding this rank's experts."""
        cfg = self.config
        E = cfg.num_moe_experts
        ep = ps.get_world_size('ep')
        ep_rank = ps.get_rank_in('ep') if ep > 1 else 0
        El = E // ep
        ep_prefix = f'{prefix}{self.hf_experts_prefix}.'
        fc1 = experts.linear_fc1.weight if experts is not None else None
        fc2 = experts.linear_fc2.weight if experts is not None else None
        glu = cfg.gated_linear_unit
        _, etp, etp_rank = self._group_info(True)
        n_gate, n_up, n_down = self.hf_expert_proj_names
        if to_mcore:
            if experts is None:
                return
            fused_key = ep_prefix + 'gate_up_proj'
            fused = fused_key in hf_sd or (fused_key + '.weight') in hf_sd
            if fused:
                k1 = fused_key if fused_key in hf_sd else fused_key + '.weight'
                k2 = ep_prefix + 'down_proj' if (ep_prefix + 'down_proj') in hf_sd else ep_prefix + 'down_proj.weight'
                w1 = self._load_hf(hf_sd, k1)[ep_rank * El:(ep_rank + 1) * El]
                w2 = self._load_hf(hf_sd, k2)[ep_rank * El:(ep_rank + 1) * El]
                # Output-major ``[E, 2F, H]`` / ``[E, H, F]`` or input-major ``[E, H, 2F]`` / ``[E, F, H]`` (the layout
                # of these families changed between Transformers releases): read it off whichever tensor is not square
                if w1.shape[1] != w1.shape[2]:
                    transposed = w1.shape[-1] != cfg.hidden_size
                elif w2.shape[1] != w2.shape[2]:
                    transposed = w2.shape[1] != cfg.hidden_size
                else:
                    transposed = bool(self.hf_experts_transposed)
                self._experts_transposed_seen = transposed
                if transposed:
                    w1, w2 = w1.transpose(1, 2), w2.transpose(1, 2)
            else:
                l1, l2 = [], []
                for e in range(ep_rank * El, (ep_rank + 1) * El):
                    p = f'{ep_prefix}{e}.'
                    if glu:
                        l1.append(torch.cat([self._load_hf(hf_sd, p + n_gate + '.weight'),
                                             self._load_hf(hf_sd, p + n_up + '.weight')], dim=0))
                    else:
                        l1.append(self._load_hf(hf_sd, p + n_up + '.weight'))
                    l2.append(self._load_hf(hf_sd, p + n_down + '.weight'))
                w1, w2 = torch.stack(l1), torch.stack(l2)
            w1s = torch.stack([shard(w1[i], 'glu' if glu else 0, etp_rank, etp) for i in range(El)])
            w2s = torch.stack([shard(w2[i], 1, etp_rank, etp) for i in range(El)])
            with torch.no_grad():
                fc1.copy_(w1s.to(device=fc1.device, dtype=fc1.dtype))
                fc2.copy_(w2s.to(device=fc2.device, dtype=fc2.dtype))
        else:
            if not self._agree(experts is not None, self._device):
                return

            def gather(p, tp_dim):
                t = None if p is None else p.detach()
                if t is not None and etp > 1:
                    parts = [torch.empty_like(t) for _ in range(etp)]
                    dist.all_gather(parts, t.contiguous(), group=ps.get_group('etp'))
                    t = torch.stack([unshard([q[i] for q in parts], tp_dim) for i in range(t.shape[0])])
                t = self._all_gather_ep(t)
                return self._broadcast_pp(t, self._device)

            w1, w2 = gather(fc1, 'glu' if glu else 0), gather(fc2, 1)
            if w1 is None:
                return
            if self.hf_fused_experts:
                if getattr(self, '_experts_transposed_seen', self.hf_experts_transposed):
                    w1, w2 = w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous()
                self._emit(hf_sd, ep_prefix + 'gate_up_proj', w1)
                self._emit(hf_sd, ep_prefix + 'down_proj', w2)
                return
            for e in range(E):
                p = f'{ep_prefix}{e}.'
                if glu:
                    g, u = w1[e].chunk(2, dim=0)
                    self._emit(hf_sd, p + n_gate + '.weight', g)
                    self._emit(hf_sd, p + n_up + '.weight', u)
                else:
                    self._emit(hf_sd, p + n_up + '.weight', w1[e])
                self._emit(hf_sd, p + n_down + '.weight', w2[e])

    def _set_moe(self, mlp, hf_sd, prefix: str, to_mcore: bool):
        cfg = self.config
        router = mlp.router if mlp is not None else None
        self._direct(router, 'weight', hf_sd, prefix + self.hf_gate_key, to_mcore)
        if cfg.moe_n_hash_layers:
            # hash-routed layers carry the token-id -> experts table next to the gate
            hashed = router if (router is not None and getattr(router, 'is_hash_layer', False)) else None
            self._direct(hashed, 'tid2eid', hf_sd, prefix + self.hf_gate_key.rsplit('.', 1)[0] + '.tid2eid', to_mcore)
        if cfg.moe_router_enable_expert_bias:
            self._direct(router, 'expert_bias', hf_sd, prefix + self.hf_expert_bias_key, to_mcore, optional=True,
                         to_mg=lambda w: w.reshape(-1),
                         to_hf=(lambda w: w.reshape(1, -1)) if self.hf_expert_bias_2d else None)
        self._set_experts(mlp.experts if mlp is not None else None, hf_sd, prefix, to_mcore)
        if cfg.moe_shared_expert_intermediate_size:
            sh = mlp.shared_experts if mlp is not None else None
            self._set_dense_mlp(sh, hf_sd, f'{prefix}{self.hf_shared_expert_prefix}.', to_mcore)
            if cfg.moe_shared_expert_gate:
                self._direct(sh, 'gate_weight', hf_sd, prefix + self.hf_shared_expert_gate_key, to_mcore)

    def _layer_is_moe(self, layer_idx: int) -> bool:
        cfg = self.config
        return bool(cfg.num_moe_experts) and bool(cfg.moe_layer_pattern()[min(layer_idx, cfg.num_layers - 1)])

    def _set_layer_mlp(self, layer, hf_sd, prefix: str, layer_idx: int, to_mcore: bool):
        mp = f'{prefix}{self.hf_mlp_prefix}.'
        mlp = layer.mlp if layer is not None else None
        if self._layer_is_moe(layer_idx):
            self._direct(layer, 'pre_mlp_layernorm.weight', hf_sd, prefix + self.hf_post_attention_layernorm_key,
                         to_mcore)
            self._set_moe(mlp, hf_sd, mp, to_mcore)
        else:
            self._direct(mlp, 'linear_fc1.layer_norm_weight', hf_sd, prefix + self.hf_post_attention_layernorm_key,
                         to_mcore)
            self._set_dense_mlp(mlp, hf_sd, mp, to_mcore)

    def _set_hyper_connection(self, hc, hf_sd, prefix: str, name: str, to_mcore: bool):
        """One hyper-connection module <-> ``hc_{name}_fn`` (projection), ``hc_{name}_base`` (bias) and
        ``hc_{name}_scale`` (the scales stacked ``[pre, post, res]``; the block's output contraction has only the
        first).  Parity: reference ``src/mcore_bridge/bridge/gpt_bridge.py:1653-1673``."""
        self._direct(hc, 'mapping_proj.weight', hf_sd, f'{prefix}hc_{name}_fn', to_mcore)
        self._direct(hc, 'bias', hf_sd, f'{prefix}hc_{name}_base', to_mcore)
        alphas = ['alpha_pre', 'alpha_post', 'alpha_res'] if name != 'head' else ['alpha_pre']
        key = f'{prefix}hc_{name}_scale'
        if to_mcore:
            if hc is None:
                return
            scale = self._load_hf(hf_sd, key).reshape(-1)
            with torch.no_grad():
                for i, a in enumerate(alphas):
                    getattr(hc, a).copy_(scale[i:i + 1].to(getattr(hc, a).dtype))
            return
        if not self._agree(hc is not None, self._device):
            return
        local = None if hc is None else torch.cat([getattr(hc, a).detach().reshape(1) for a in alphas])
        self._emit(hf_sd, key, self._broadcast_pp(local, self._device))

    def _set_layer_state(self, layer, hf_sd, prefix: str, layer_idx: int, to_mcore: bool):
        self._set_layer_attn(layer, hf_sd, prefix, to_mcore)
        self._set_layer_mlp(layer, hf_sd, prefix, layer_idx, to_mcore)
        if self.config.enable_hyper_connections:
            self._set_hyper_connection(getattr(layer, 'self_attention_hyper_connection', None) if layer is not None
                                       else None, hf_sd, prefix, 'attn', to_mcore)
            self._set_hyper_connection(getattr(layer, 'mlp_hyper_connection', None) if layer is not None else None,
                                       hf_sd, prefix, 'ffn', to_mcore)

    # ------------------------------------------------------------------ walker
    def _find_layer(self, mg_models: List[nn.Module], layer_idx: int):
        for m in mg_models:
            dec = m.decoder
            off = dec.layer_offset
            if off <= layer_idx < off + len(dec.layers):
                return dec.layers[layer_idx - off]
        return None

    def _convert(self, mg_models: List[nn.Module], hf_sd: Dict[str, Any], to_mcore: bool, tqdm_desc: str = ''):
        """Drives all slots.  Load: fills the model, yields nothing.  Export: yields ``(hf_key, tensor)``."""
        from ..utils.megatron_utils import unwrap_model
        wrappers = unwrap_model(list(mg_models))
        mg_models = [self._language_model(m) for m in wrappers]
        cfg = self.config
        first = next((m for m in mg_models if getattr(m, 'pre_process', False)), None)
        last = next((m for m in mg_models if getattr(m, 'post_process', False)), None)
        out: Dict[str, torch.Tensor] = hf_sd if to_mcore else {}

        def flush():
            items = list(out.items())
            out.clear()
            return items

        self._convert_pre_process(first, out, to_mcore)
        if not to_mcore:
            yield from flush()
        self._convert_hf_modules(wrappers, out, to_mcore)
        if not to_mcore:
            yield from flush()
        layer_iter: Iterable[int] = range(cfg.num_layers)
        if tqdm_desc and is_master():
            try:
                from tqdm import tqdm
                layer_iter = tqdm(layer_iter, desc=tqdm_desc, dynamic_ncols=True)
            except Exception:
                pass
        for i in layer_iter:
            layer = self._find_layer(mg_models, i)
            if to_mcore and layer is None:
                continue
            self._set_layer_state(layer, out, f'{self.hf_layers_prefix}.{i}.', i, to_mcore)
            if not to_mcore:
                yield from flush()
        if cfg.mtp_num_layers:
            self._convert_mtp(last, out, to_mcore)
            if not to_mcore:
                yield from flush()
        self._convert_post_process(last, out, to_mcore)
        if not to_mcore:
            yield from flush()

    def _find_tower(self, wrappers):
        for m in wrappers:
            while hasattr(m, 'base_model') or (hasattr(m, 'model') and not hasattr(m, 'language_model')
                                               and not hasattr(m, 'decoder')):
                m = m.base_model if hasattr(m, 'base_model') else m.model
            tower = getattr(m, 'visual', None)
            if tower is not None:
                return tower
        return None

    def _convert_hf_modules(self, wrappers, hf_sd, to_mcore: bool):
        """Media towers keep their Hugging Face parameter names: each ``module_mapping`` entry (HF prefix ->
        attribute of the tower wrapper) is copied tensor by tensor.  Towers are replicated over TP and live on
        the first pipeline stage; on export that stage's ranks publish the key list so the others can take part
        in the broadcasts.  Parity: reference ``src/mcore_bridge/bridge/gpt_bridge.py:2009-2042``."""
        meta = self.config.model_meta
        if getattr(meta, 'visual_cls', None) is None or self.config.language_model_only:
            return
        tower = self._find_tower(wrappers)
        mapping = dict(meta.visual_cls.module_mapping)
        if to_mcore:
            if tower is None:
                return
            for hf_prefix, attr in mapping.items():
                sub = deep_getattr(tower, attr)
                if sub is None:               # optional tower the config leaves out (e.g. no audio encoder)
                    continue
                state = sub.state_dict(keep_vars=True)
                for name, t in state.items():
                    key = f'{hf_prefix}.{name}'
                    if key not in hf_sd:
                        if isinstance(t, nn.Parameter):
                            raise KeyError(f'{key} is missing from the checkpoint')
                        continue              # non-persistent-like buffers recomputed at construction
                    with torch.no_grad():
                        t.copy_(self._load_hf(hf_sd, key).to(dtype=t.dtype, device=t.device))
            return
        names = None
        if tower is not None:
            names = []
            for hf_prefix, attr in mapping.items():
                sub = deep_getattr(tower, attr)
                if sub is None:
                    continue
                names += [(f'{hf_prefix}.{n}', attr, n) for n in sub.state_dict().keys()]
        if ps.get_world_size('pp') > 1:
            box = [None] * ps.get_world_size('pp')
            dist.all_gather_object(box, names, group=ps.get_group('pp'))
            names = next((b for b in box if b is not None), None)
        for key, attr, n in names or []:
            t = None
            if tower is not None:
                t = deep_getattr(tower, attr).state_dict(keep_vars=True)[n].detach()
            self._emit(hf_sd, key, self._broadcast_pp(t, self._device))

    def _language_model(self, m):
        while hasattr(m, 'base_model') or (hasattr(m, 'model') and not hasattr(m, 'decoder')):
            m = m.base_model if hasattr(m, 'base_model') else m.model   # strip PEFT wrappers
        return getattr(m, 'language_model', m)

    def _convert_modules_to_save(self, model, adapter_name: str):
        """Trainable copies made by ``modules_to_save`` (embedding / head / final norm), under their HF keys."""
        from ..tuners.peft_model import ModulesToSaveWrapper
        out: Dict[str, torch.Tensor] = {}
        rows, actual = self._vocab_rows(), self.config.padded_vocab_size
        emb = getattr(getattr(model, 'embedding', None), 'word_embeddings', None)
        if isinstance(emb, ModulesToSaveWrapper):
            self._direct(emb, 'weight', out, self.hf_embed_key, False, tp_dim=0, to_hf=lambda w: w[:actual])
        if isinstance(getattr(model, 'output_layer', None), ModulesToSaveWrapper):
            self._direct(model.output_layer, 'weight', out, self.hf_lm_head_key, False, tp_dim=0,
                         to_hf=lambda w: w[:actual])
        dec = getattr(model, 'decoder', None)
        if dec is not None and isinstance(getattr(dec, 'final_layernorm', None), ModulesToSaveWrapper):
            self._direct(dec.final_layernorm, 'weight', out, self.hf_final_layernorm_key, False)
        yield from out.items()

    def _convert_mtp(self, model, hf_sd, to_mcore: bool):
        """Multi-token-prediction layers are stored after the decoder layers (``model.layers.{L + k}``) with
        ``enorm`` / ``hnorm`` / ``eh_proj`` and an ordinary transformer layer (DeepSeek-V3 convention)."""
        cfg = self.config
        mtp = model.mtp if (model is not None and getattr(model, 'mtp', None) is not None) else None
        if to_mcore and mtp is not None and not getattr(model, 'pre_process', False) \
                and getattr(model, 'embedding', None) is not None:
            # under pipeline parallelism the last stage looks the MTP depths' tokens up in an embedding of its own:
            # a second copy of the first stage's matrix
            rows = self._vocab_rows()
            self._direct(model.embedding.word_embeddings, 'weight', hf_sd, self.hf_embed_key, True, tp_dim=0,
                         to_mg=lambda w: self._pad_vocab(w, rows))
        for k in range(cfg.mtp_num_layers):
            prefix = f'{self.hf_layers_prefix}.{cfg.num_layers + k}.'
            lay = mtp.layers[k] if mtp is not None else None
            if to_mcore and (lay is None or (prefix + 'eh_proj.weight') not in hf_sd):
                if lay is not None:
                    logger.warning_once('the checkpoint has no MTP weights; MTP layers keep their initialisation')
                continue
            self._direct(lay, 'enorm.weight', hf_sd, prefix + 'enorm.weight', to_mcore)
            self._direct(lay, 'hnorm.weight', hf_sd, prefix + 'hnorm.weight', to_mcore)
            self._direct(lay, 'eh_proj.weight', hf_sd, prefix + 'eh_proj.weight', to_mcore, tp_dim=0)
            self._direct(lay, 'final_layernorm.weight', hf_sd, prefix + 'shared_head.norm.weight', to_mcore)
            self._set_layer_state(lay.transformer_layer if lay is not None else None, hf_sd, prefix,
                                  cfg.num_layers - 1, to_mcore)

    # ------------------------------------------------------------------ public API
    def load_weights(self, mg_models, hf_model_dir: str, peft_format: bool = False, adapter_name: str = 'default',
                     converter: Optional[Callable] = None) -> None:
        self._peft_format, self._adapter_name = peft_format, adapter_name
        if not isinstance(mg_models, (list, tuple)):
            mg_models = [mg_models]
        with SafetensorLazyLoader(hf_model_dir, peft_format=peft_format) as loader:
            sd = loader.get_state_dict()
            if not peft_format:
                sd = add_dequantized_views(sd, self._quantization_config(hf_model_dir), LazyTensor)
            if converter is not None:
                sd = {k2: v2 for k, v in sd.items() for k2, v2 in self._apply_converter(converter, k, v)}
            if (self.hf_state_dict_mapping or self.hf_load_aliases) and not peft_format:
                sd = {self._modernise_key(k): v for k, v in sd.items()}
            if peft_format:
                from .peft_bridge import load_adapter
                sd = {self._peft_key(k, True): v for k, v in sd.items()}
                load_adapter(self, mg_models, sd, adapter_name)
            else:
                for _ in self._convert(mg_models, sd, True, tqdm_desc='Loading: '):
                    pass
        self._peft_format = False

    def _quantization_config(self, hf_model_dir: str) -> Optional[dict]:
        """``quantization_config`` of the checkpoint: from the model's Hugging Face config, else from the directory."""
        qc = getattr(self.config.hf_config, 'quantization_config', None)
        if qc is None:
            import json
            import os
            path = os.path.join(hf_model_dir, 'config.json')
            if os.path.exists(path):
                with open(path, 'r', encoding='utf-8') as f:
                    cfg = json.load(f)
                qc = cfg.get('quantization_config') or (cfg.get('text_config') or {}).get('quantization_config')
        if qc is not None and not isinstance(qc, dict):
            qc = qc.to_dict() if hasattr(qc, 'to_dict') else dict(qc)
        return qc

    def _legacy_key(self, key: str) -> str:
        """Inverse of ``_modernise_key``: such checkpoints are written in the layout they are published in."""
        for old, new in self.hf_state_dict_mapping.items():
            if key.startswith(new + '.'):
                return old + key[len(new):]
        return key

    def _modernise_key(self, key: str) -> str:
        for old, new in {**self.hf_state_dict_mapping, **self.hf_load_aliases}.items():
            if key.startswith(old + '.') and not key.startswith(new + '.'):
                return new + key[len(old):]
        return key

    def _peft_key(self, key: str, to_mcore: bool) -> str:
        """Adapter key as stored on disk <-> the name used internally; families whose checkpoint names differ from
        the internal ones override it."""
        return key

    def _peft_layer_slots(self, layer_idx: int):
        """Adapter slot table of one layer for families whose layers differ from the generic ones (``None``: the generic
        table of ``peft_bridge._layer_slots``).  Entries: (path inside the layer, kind, Hugging Face prefix relative to
        the layer, Hugging Face module names); kind ``custom_col`` re-lays ``lora_B`` through ``_peft_split`` /
        ``_peft_join``."""
        return None

    def _peft_model_slots(self):
        """``(slots, Hugging Face prefix)`` of wrapped linears that belong to the model, not to a layer."""
        return None

    def _peft_split(self, layer_prefix: str, path: str, B: torch.Tensor, names):
        raise NotImplementedError

    def _peft_join(self, layer_prefix: str, path: str, parts, names) -> torch.Tensor:
        raise NotImplementedError

    def _peft_module_name(self, name: str) -> str:
        """Internal linear name -> the name ``adapter_config.json`` lists under ``target_modules``."""
        return name

    @staticmethod
    def _apply_converter(converter, key, value):
        res = converter(key, value)
        if res is None:
            return []
        if isinstance(res, tuple) and len(res) == 2 and isinstance(res[0], str):
            return [res]
        return list(res)

    def export_weights(self, mg_models, target_device=None, only_master_rank: bool = False, peft_format: bool = False,
                       adapter_name: str = 'default', converter: Optional[Callable] = None,
                       tqdm_desc: str = 'Exporting: '):
        self._target_device, self._only_master_rank = target_device, only_master_rank
        self._peft_format, self._adapter_name = peft_format, adapter_name
        if not isinstance(mg_models, (list, tuple)):
            mg_models = [mg_models]
        from ..train.distributed_optimizer import finish_all_param_gathers
        finish_all_param_gathers()        # an overlapped parameter all-gather may still be writing the weights
        try:
            if peft_format:
                from .peft_bridge import export_adapter
                gen = export_adapter(self, mg_models, adapter_name)
            else:
                gen = self._convert(mg_models, {}, False, tqdm_desc=tqdm_desc)
            with torch.no_grad():
                for k, v in gen:
                    if self.hf_state_dict_mapping and not peft_format:
                        k = self._legacy_key(k)
                    elif peft_format:
                        k = self._peft_key(k, False)
                    if converter is not None:
                        for k2, v2 in self._apply_converter(converter, k, v):
                            yield k2, v2
                    else:
                        yield k, v
        finally:
            self._target_device, self._only_master_rank, self._peft_format = None, False, False

    def save_weights(self, mg_models, output_dir: str, peft_format: bool = False, adapter_name: str = 'default',
                     converter: Optional[Callable] = None, max_shard_size: str = '5GB') -> None:
        saver = StreamingSafetensorSaver(output_dir, max_shard_size=max_shard_size, peft_format=peft_format)
        for k, v in self.export_weights(mg_models, target_device='cpu', only_master_rank=True,
                                        peft_format=peft_format, adapter_name=adapter_name, converter=converter,
                                        tqdm_desc='Saving: '):
            saver.add_tensor(k, v)
        saver.finalize()
        targets = None
        if peft_format:
            # the names are collected over the pipeline group: every rank takes part, only the master writes
            from .peft_bridge import hf_target_modules
            targets = hf_target_modules(self, mg_models if isinstance(mg_models, (list, tuple)) else [mg_models],
                                        adapter_name)
            targets = sorted({self._peft_module_name(t) for t in targets})
        if is_master():
            self._save_config(output_dir, peft_format, mg_models, adapter_name, targets)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()

    def _save_config(self, output_dir: str, peft_format: bool, mg_models, adapter_name: str, target_modules=None):
        if peft_format:
            from .peft_bridge import save_adapter_config
            save_adapter_config(self, mg_models if isinstance(mg_models, (list, tuple)) else [mg_models], output_dir,
                                adapter_name, target_modules)
            return
        hf_config = self.config.hf_config
        if hf_config is not None and hasattr(hf_config, 'save_pretrained'):
            hf_config.save_pretrained(output_dir)


class MultimodalGPTBridge(GPTBridge):
    """Bridge for models whose language model sits under ``language_model`` next to HF vision modules
    (parity: reference ``src/mcore_bridge/bridge/gpt_bridge.py:2062-2065``)."""
    hf_layers_prefix = 'model.language_model.layers'
    hf_embed_key = 'model.language_model.embed_tokens.weight'
    hf_final_layernorm_key = 'model.language_model.norm.weight'
