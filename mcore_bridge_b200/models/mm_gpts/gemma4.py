"""Gemma-4: text decoder (``gemma4_text``), the multimodal wrapper (``gemma4``) and the weight bridge.

What differs from the generic decoder, all of it read from the Hugging Face text config:

* two layer types with their own head size, KV-head count and rope table — ``sliding_attention`` (``head_dim``,
  plain rope, windowed) and ``full_attention`` (``global_head_dim``, "proportional" rope that rotates only the first
  part of the head, optionally ``attention_k_eq_v``: no value projection, values are the un-normalised keys);
* q / k RMSNorm with weights, v RMSNorm without, softmax scale 1;
* the last ``num_kv_shared_layers`` layers project queries only and attend to the keys / values of the last
  non-shared layer of their type; their dense MLP may be twice as wide (``use_double_wide_mlp``);
* sandwich norms around attention and MLP, an optional MoE branch that runs beside the dense MLP (router fed with
  the un-normalised residual, experts with its own pre-norm, one post-norm per branch), an optional per-layer input
  path (a second embedding table plus a projection of the word embeddings, gated into every layer) and a
  ``layer_scalar`` buffer multiplied into the layer output;
* word embeddings scaled by ``sqrt(hidden)``, logits soft-capped with ``tanh``.

Parity: reference ``src/mcore_bridge/model/mm_gpts/gemma4.py`` (attention 139-361, MLP / MoE 364-418, bridge
421-509, model 512-711, layer 714-819, tower 58-136).  Under pipeline parallelism the per-layer inputs and the shared
keys / values are packed behind the hidden states sent to the next stage (reference 656-703).  Limits: global
layers with a head size above 256 use the masked-softmax attention path.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ...bridge.gpt_bridge import MultimodalGPTBridge
from ...layers.context import ForwardContext
from ...layers.embedding import VocabParallelEmbedding
from ...layers.linear import ColumnParallelLinear, LayerNormColumnParallelLinear, RowParallelLinear
from ...layers.mlp import MLP
from ...layers.moe import MoELayer
from ...layers.norm import Norm, mark_sequence_parallel
from ...ops.attention import attention
from ...ops.cross_entropy import vocab_parallel_cross_entropy
from ...ops.linear import LinearSpec, linear
from ...ops.rope import apply_rope
from ...parallel import mappings as M
from ...parallel import state as ps
from ...utils.logger import get_logger
from ...utils.utils import deep_getattr
from ..constant import ModelType
from ..gpt_model import GPTModel
from ..mm_gpt_model import MultimodalGPTModel
from ..register import ModelLoader, ModelMeta, register_model
from ..transformer_block import TransformerBlock
from .base import HuggingFaceVit

logger = get_logger()
SHARED_KV = 'gemma4_shared_kv'          # ctx.extra: layer type -> (k, v) of the last non-shared layer of that type
PER_LAYER = 'gemma4_per_layer_inputs'   # ctx.extra: [T, L, P] per-layer input vectors


def text_config_of(config):
    hf = config.hf_config
    return getattr(hf, 'text_config', None) or hf


def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm without a weight, computed in fp32."""
    xf = x.float()
    return (xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)).to(x.dtype)


def layer_kinds(tc, num_layers: int):
    """Per layer: (type, head_dim, kv_heads, k_eq_v, is_kv_shared, stores_kv)."""
    first_shared = num_layers - (getattr(tc, 'num_kv_shared_layers', 0) or 0)
    prev = list(tc.layer_types[:first_shared])
    out = []
    for i in range(num_layers):
        lt = tc.layer_types[i]
        sliding = lt == 'sliding_attention'
        d = tc.global_head_dim if (not sliding and tc.global_head_dim) else tc.head_dim
        k_eq_v = bool(tc.attention_k_eq_v) and not sliding
        ng = tc.num_global_key_value_heads if k_eq_v else tc.num_key_value_heads
        shared = i >= first_shared > 0
        stores = False
        if not shared and first_shared < num_layers and lt in prev:
            stores = i == len(prev) - 1 - prev[::-1].index(lt)
        out.append((lt, d, ng, k_eq_v, shared, stores))
    return out


class Gemma4Rope(nn.Module):
    """cos / sin tables ``[T, d/2]`` for one layer type (default or proportional frequencies)."""

    def __init__(self, tc, layer_type: str):
        super().__init__()
        rp = dict(tc.rope_parameters[layer_type])
        kind = rp.get('rope_type', 'default')
        base = rp['rope_theta']
        if kind == 'default':
            d = tc.head_dim
            inv = 1.0 / (base ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
            scale = 1.0
        elif kind == 'proportional':
            d = (tc.global_head_dim if layer_type == 'full_attention' else None) or tc.head_dim
            angles = int(rp.get('partial_rotary_factor', 1.0) * d // 2)
            inv = 1.0 / (base ** (torch.arange(0, 2 * angles, 2, dtype=torch.int64).float() / d))
            inv = torch.cat([inv, torch.zeros(d // 2 - angles)]) / rp.get('factor', 1.0)
            scale = 1.0
        else:       # the scaled variants keep their Transformers definition
            from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
            inv, scale = ROPE_INIT_FUNCTIONS[kind](tc, None, layer_type=layer_type)
        self.register_buffer('inv_freq', inv.float(), persistent=False)
        self.attention_scaling = float(scale)

    def forward(self, positions: torch.Tensor):
        f = positions.to(self.inv_freq.device).float()[:, None] * self.inv_freq[None, :]
        return f.cos() * self.attention_scaling, f.sin() * self.attention_scaling


class Gemma4Attention(nn.Module):
    """``linear_qkv`` rows are grouped per KV head as ``[q heads of the group | k | v]`` (``[q | k]`` with
    ``attention_k_eq_v``; query heads only on a KV-shared layer), so a TP shard is a whole number of groups."""

    def __init__(self, config, layer_number: int):
        super().__init__()
        self.config = config
        tc = text_config_of(config)
        (self.layer_type, self.d, self.ng, self.k_eq_v, self.is_kv_shared,
         self.stores_kv) = layer_kinds(tc, config.num_layers)[layer_number - 1]
        tp = ps.get_world_size('tp')
        self.nq = config.num_attention_heads
        if self.nq % tp:
            raise NotImplementedError(f'Gemma-4 attention needs query heads ({self.nq}) divisible by TP {tp}')
        # More TP ranks than KV heads: the row split of ``linear_qkv`` cuts through a group, so the projection output is
        # all-gathered on the last dim and every rank takes its group and, inside it, its share of the query heads;
        # ``kv_rep`` ranks then share one KV head (reference
        # ``src/mcore_bridge/model/mm_gpts/gemma4.py:305-309,343-346``)
        self.kv_rep = 1
        if self.ng % tp:
            if tp % self.ng:
                raise NotImplementedError(f'TP ({tp}) must divide or be a multiple of the KV heads ({self.ng})')
            self.kv_rep = tp // self.ng
        self.nq_local, self.ng_local, self.qpg = self.nq // tp, max(1, self.ng // tp), self.nq // self.ng
        self.kv_per_group = 0 if self.is_kv_shared else (1 if self.k_eq_v else 2)
        out = (self.nq + self.ng * self.kv_per_group) * self.d
        self.linear_qkv = LayerNormColumnParallelLinear(config.hidden_size, out, config, bias=config.add_qkv_bias)
        self.q_layernorm = Norm(config, self.d, sequence_parallel_grad=False)
        self.k_layernorm = None if self.is_kv_shared else Norm(config, self.d, sequence_parallel_grad=False)
        for n_ in (self.q_layernorm, self.k_layernorm):
            if n_ is not None:      # replicated weight applied to local heads: partial gradients, summed over TP
                n_.weight.sequence_parallel = tp > 1
        self.window = (int(tc.sliding_window) - 1, 0) if self.layer_type == 'sliding_attention' else None
        self.linear_proj = RowParallelLinear(self.nq * self.d, config.hidden_size, config, bias=config.add_bias_linear)

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        eps = self.config.layernorm_epsilon
        qkv = self.linear_qkv(x)
        T = qkv.shape[0]
        cos, sin = ctx.rope_tables[self.layer_type]
        shared = ctx.extra.setdefault(SHARED_KV, {})
        if self.is_kv_shared:
            q = qkv.view(T, self.nq_local, self.d)
            k, v = shared[self.layer_type]
        else:
            if self.kv_rep > 1:
                r = ps.get_rank_in('tp')
                gsize = (self.qpg + self.kv_per_group) * self.d
                full = M.all_gather_last_dim_sum_grad(qkv, 'tp')
                g = full[:, (r // self.kv_rep) * gsize:(r // self.kv_rep + 1) * gsize].view(
                    T, 1, self.qpg + self.kv_per_group, self.d)
                q0 = (r % self.kv_rep) * self.nq_local
                q = g[:, 0, q0:q0 + self.nq_local]
            else:
                g = qkv.view(T, self.ng_local, self.qpg + self.kv_per_group, self.d)
                q = g[:, :, :self.qpg].reshape(T, self.nq_local, self.d)
            k_raw = g[:, :, self.qpg]
            v_raw = k_raw if self.k_eq_v else g[:, :, self.qpg + 1]
            k = apply_rope(self.k_layernorm(k_raw.contiguous()), cos, sin, False)
            v = _rms(v_raw, eps).contiguous()
            if self.stores_kv:
                shared[self.layer_type] = (k, v)
        q = apply_rope(self.q_layernorm(q.contiguous()), cos, sin, False)
        if ps.get_world_size('cp') > 1:
            raise NotImplementedError('Gemma-4 attention does not run under context parallelism')
        o = attention(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, causal=True, scale=1.0, window=self.window,
                      seq_start=ctx.seq_start)
        return self.linear_proj(o.reshape(T, -1))


class Gemma4MoE(MoELayer):
    """Routed experts running beside the dense MLP.  The router sees the residual stream through a weight-less
    RMSNorm, a learned per-channel ``scale`` and ``hidden**-0.5``; the selected probabilities are renormalised
    and multiplied by ``per_expert_scale``; the experts see the residual through ``pre_feedforward_layernorm_2``."""

    def __init__(self, config, layer_number: int = 1):
        super().__init__(config, layer_number)
        h = config.hidden_size
        self.pre_feedforward_layernorm_2 = Norm(config, h)
        self.scale = nn.Parameter(torch.ones(h, dtype=config.params_dtype))
        self.per_expert_scale = nn.Parameter(torch.ones(config.num_moe_experts, dtype=config.params_dtype))
        mark_sequence_parallel(self.scale, config)
        mark_sequence_parallel(self.per_expert_scale, config)
        self.scalar_root_size = h ** -0.5
        self._residual = None

    def _router_input(self, x):
        r = self._residual
        return (_rms(r, self.config.layernorm_epsilon).float() * self.scale.float() * self.scalar_root_size).to(r.dtype)

    def _post_route(self, probs, idx):
        return probs * self.per_expert_scale.float()[idx.long()].to(probs.dtype)

    def forward(self, residual, padding_mask=None, seg_ids=None, num_seqs=None):
        self._residual = residual
        try:
            return super().forward(self.pre_feedforward_layernorm_2(residual), padding_mask, seg_ids, num_seqs)
        finally:
            self._residual = None


class Gemma4Layer(nn.Module):

    def __init__(self, config, layer_number: int, is_mtp_layer: bool = False):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        tc = text_config_of(config)
        h = config.hidden_size
        kinds = layer_kinds(tc, config.num_layers)[layer_number - 1]
        self.self_attention = Gemma4Attention(config, layer_number)
        self.post_attention_layernorm = Norm(config, h)
        wide = 2 if (getattr(tc, 'use_double_wide_mlp', False) and kinds[4]) else 1
        self.mlp = MLP(config, ffn_hidden_size=config.ffn_hidden_size * wide, fuse_input_norm=True)
        self.post_feedforward_layernorm = Norm(config, h)
        self.is_moe = bool(getattr(tc, 'enable_moe_block', False))
        if self.is_moe:
            self.experts_mlp = Gemma4MoE(config, layer_number)
            self.post_feedforward_layernorm_1 = Norm(config, h)
            self.post_feedforward_layernorm_2 = Norm(config, h)
        self.per_layer_dim = int(getattr(tc, 'hidden_size_per_layer_input', 0) or 0)
        if self.per_layer_dim:
            self.per_layer_input_gate = ColumnParallelLinear(h, self.per_layer_dim, config, bias=False)
            self.per_layer_projection = RowParallelLinear(self.per_layer_dim, h, config, bias=False)
            self.post_per_layer_input_norm = Norm(config, h)
        self.act = torch.nn.functional.gelu if tc.hidden_activation == 'gelu_pytorch_tanh' else None
        if self.act is None:
            from transformers.activations import ACT2FN
            self._act_fn = ACT2FN[tc.hidden_activation]
        self.register_buffer('layer_scalar', torch.ones(1, dtype=config.params_dtype))

    def _activation(self, x):
        return torch.nn.functional.gelu(x, approximate='tanh') if self.act is not None else self._act_fn(x)

    def forward(self, hidden: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        hidden = hidden + self.post_attention_layernorm(self.self_attention(hidden, ctx))
        residual = hidden
        out = self.mlp(hidden)
        if self.is_moe:
            out = self.post_feedforward_layernorm_1(out) + self.post_feedforward_layernorm_2(
                self.experts_mlp(residual, ctx.padding_mask, ctx.seg_ids, ctx.num_seqs))
        hidden = residual + self.post_feedforward_layernorm(out)
        if self.per_layer_dim:
            pli = ctx.extra[PER_LAYER][:, self.layer_number - 1]           # [T, P / tp]: this rank's columns
            g = self._activation(self.per_layer_input_gate(hidden)) * pli.to(hidden.dtype)
            hidden = hidden + self.post_per_layer_input_norm(self.per_layer_projection(g))
        return hidden * self.layer_scalar.to(hidden.dtype)


class Gemma4Block(TransformerBlock):
    layer_cls = Gemma4Layer


class Gemma4TextModel(GPTModel):
    block_cls = Gemma4Block
    extra_forward_keys = ['mm_token_type_ids']

    def __init__(self, config, pre_process: bool = True, post_process: bool = True, vp_stage: Optional[int] = None):
        tc = text_config_of(config)
        self.per_layer_dim = int(getattr(tc, 'hidden_size_per_layer_input', 0) or 0)
        self.kv_shared_layers = int(getattr(tc, 'num_kv_shared_layers', 0) or 0)
        if getattr(tc, 'use_bidirectional_attention', None) == 'vision':
            # image tokens would attend to each other in both directions; the attention kernels here are causal
            logger.warning('use_bidirectional_attention="vision" is not supported: image tokens attend causally')
        super().__init__(config, pre_process, post_process, vp_stage)
        self.rotary_pos_emb = None
        self._received, self._ctx = None, None
        self.ropes = nn.ModuleDict({lt: Gemma4Rope(tc, lt) for lt in sorted(set(tc.layer_types))})
        self.embed_scale = float(config.hidden_size) ** 0.5
        self.final_logit_softcapping = getattr(tc, 'final_logit_softcapping', None)
        if self.per_layer_dim and pre_process:
            tp = ps.get_world_size('tp')
            total = config.num_layers * self.per_layer_dim
            rows = (tc.vocab_size_per_layer_input + tp - 1) // tp * tp
            self.embed_tokens_per_layer = VocabParallelEmbedding(rows, total, config)
            self.per_layer_model_projection = ColumnParallelLinear(config.hidden_size, total, config, bias=False,
                                                                   gather_output=True, sequence_parallel=False)
            # applied to values that are replicated over the tensor-parallel ranks and receives the full gradient on
            # each of them (see _per_layer_inputs): its weight gradient must not be summed over the group
            self.per_layer_projection_norm = Norm(config, self.per_layer_dim, sequence_parallel_grad=False)

    def build_context(self, input_ids, position_ids, attention_mask, packed_seq_params, batch, seq, device):
        ctx = super().build_context(input_ids, position_ids, attention_mask, packed_seq_params, batch, seq, device)
        pos = ctx.position_ids
        for lt, rope in self.ropes.items():
            ctx.rope_tables[lt] = rope(pos.to(device))
        if self._received is not None:          # what the previous pipeline stage sent along with the hidden states
            ctx.extra.update(self._received)
            self._received = None
        self._ctx = ctx
        return ctx

    # ---- pipeline parallelism: per-layer inputs and shared keys / values travel behind the hidden states
    def _kv_slots(self):
        """(layer type, local kv heads, head dim) of every layer type whose keys / values later layers reuse."""
        if not self.kv_shared_layers:
            return []
        tc, tp = text_config_of(self.config), ps.get_world_size('tp')
        slots = {}
        for lt, d, ng, _, _, stores in layer_kinds(tc, self.config.num_layers):
            if stores:
                slots[lt] = (lt, max(1, ng // tp), d)
        return [slots[k] for k in sorted(slots)]

    def _extra_columns(self) -> int:
        """Columns per *token* that ride along (this rank's share under tensor parallelism)."""
        tp = ps.get_world_size('tp')
        cols = self.config.num_layers * (self.per_layer_dim // tp) if self.per_layer_dim else 0
        return cols + sum(2 * h * d for _, h, d in self._kv_slots())

    def pipeline_width(self) -> int:
        """Width of the tensor exchanged between stages.  Its rows are this rank's hidden-state rows (a 1/tp slice
        of the tokens under sequence parallelism) while the extras cover all tokens, so they take tp times their
        per-token width."""
        return self.config.hidden_size + self._extra_columns() * self._tokens_per_row()

    def _tokens_per_row(self) -> int:
        sp = self.config.sequence_parallel and ps.get_world_size('tp') > 1
        return ps.get_world_size('tp') if sp else 1

    def _pack(self, hidden: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        rows = hidden.shape[0]
        parts = [hidden]
        if self.per_layer_dim:
            parts.append(ctx.extra[PER_LAYER].reshape(rows, -1).to(hidden.dtype))
        shared = ctx.extra.get(SHARED_KV, {})
        for lt, h, d in self._kv_slots():
            if lt in shared:
                k, v = shared[lt]
                parts += [k.reshape(rows, -1).to(hidden.dtype), v.reshape(rows, -1).to(hidden.dtype)]
            else:       # produced by a later stage: placeholders keep the width static
                parts += [hidden.new_zeros(rows, self._tokens_per_row() * h * d)] * 2
        return torch.cat(parts, dim=-1)

    def set_input_tensor(self, input_tensor):
        if isinstance(input_tensor, (list, tuple)):
            input_tensor = input_tensor[0]
        H = self.config.hidden_size
        if input_tensor is None or input_tensor.shape[-1] == H:
            return super().set_input_tensor(input_tensor)
        rows = input_tensor.shape[0]
        tokens = rows * self._tokens_per_row()
        tp = ps.get_world_size('tp')
        assert input_tensor.shape[-1] == self.pipeline_width(), (input_tensor.shape, self.pipeline_width())
        got, at = {}, H
        if self.per_layer_dim:
            w = tokens * self.config.num_layers * (self.per_layer_dim // tp) // rows
            got[PER_LAYER] = input_tensor[:, at:at + w].reshape(tokens, self.config.num_layers,
                                                                self.per_layer_dim // tp)
            at += w
        kv = {}
        for lt, h, d in self._kv_slots():
            w = tokens * h * d // rows
            kv[lt] = (input_tensor[:, at:at + w].reshape(tokens, h, d),
                      input_tensor[:, at + w:at + 2 * w].reshape(tokens, h, d))
            at += 2 * w
        if kv:
            got[SHARED_KV] = kv
        self._received = got
        super().set_input_tensor(input_tensor[:, :H])

    def forward(self, *args, **kwargs):
        out = super().forward(*args, **kwargs)
        if not self.post_process and self._extra_columns():
            out = self._pack(out, self._ctx)
        self._ctx = None
        return out

    # ---- embeddings
    def _per_layer_inputs(self, embeds_full: torch.Tensor, ids: Optional[torch.Tensor], ctx: ForwardContext):
        """``[T, L, P]``: projection of the (scaled) word embeddings, normalised per layer, averaged with the per-layer
        embedding table's row of each token."""
        L, P = self.config.num_layers, self.per_layer_dim
        proj = self.per_layer_model_projection(embeds_full)
        proj = self.per_layer_projection_norm((proj * float(self.config.hidden_size) ** -0.5).view(-1, L, P))
        if ids is not None:
            tab = self.embed_tokens_per_layer(ids.reshape(-1).clamp(min=0))
            tab = (tab * torch.tensor(float(P) ** 0.5, dtype=tab.dtype)).view(-1, L, P)
            proj = (proj + tab) * (2.0 ** -0.5)
        if ps.get_world_size('tp') > 1:
            # Every layer's gate is column-parallel over P: keep this rank's columns only.  The values were computed
            # identically on every rank, so the backward gathers the ranks' column gradients into the full gradient.
            proj = M.scatter_to_tensor_model_parallel_region(proj, 'tp')
        ctx.extra[PER_LAYER] = proj

    def embed(self, flat_ids, ctx, sp):
        e = self.embedding(flat_ids.clamp(min=0), scatter_to_sequence_parallel=False)
        e = e * torch.tensor(self.embed_scale, dtype=e.dtype)
        if self.per_layer_dim:
            self._per_layer_inputs(e, flat_ids, ctx)
        return M.scatter_to_sequence_parallel_region(e) if sp else e

    def on_decoder_input(self, hidden_full, ctx):
        # a multimodal wrapper hands over embeddings it has already scaled; the ids it passes along have the media
        # placeholders replaced by the padding id
        if self.per_layer_dim:
            ids = ctx.extra.get('llm_input_ids')
            if ids is None:
                ids = ctx.input_ids
            self._per_layer_inputs(hidden_full, ids, ctx)
        return hidden_full

    # ---- head
    def finalize_logits(self, logits):
        cap = self.final_logit_softcapping
        if cap is None:
            return logits
        return (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)

    def _lm_loss(self, hidden_full, labels_flat):
        if self.final_logit_softcapping is None:
            return super()._lm_loss(hidden_full, labels_flat)
        logits = linear(hidden_full, self._head_weight(), None, LinearSpec())
        return vocab_parallel_cross_entropy(self.finalize_logits(logits).float(), labels_flat, 'tp')


class Gemma4Model(MultimodalGPTModel):
    language_model_cls = Gemma4TextModel


# ------------------------------------------------------------------------------------------------- weight bridge
class Gemma4Bridge(MultimodalGPTBridge):
    """Key layout of ``Gemma4ForConditionalGeneration`` (``model.language_model.*``) or, for a text-only config,
    of ``Gemma4ForCausalLM`` (``model.*``)."""
    hf_fused_experts = True

    def __init__(self, config):
        super().__init__(config)
        self.tc = text_config_of(config)
        self.lm_prefix = 'model.language_model.' if hasattr(config.hf_config, 'text_config') else 'model.'
        self.hf_layers_prefix = self.lm_prefix + 'layers'
        self.hf_embed_key = self.lm_prefix + 'embed_tokens.weight'
        self.hf_final_layernorm_key = self.lm_prefix + 'norm.weight'
        self.kinds = layer_kinds(self.tc, config.num_layers)

    # q / k / v <-> rows grouped per KV head
    def _set_gemma_qkv(self, attn, hf_sd, ap: str, kind, to_mcore: bool):
        _, d, ng, k_eq_v, shared, _ = kind
        nq = self.config.num_attention_heads
        names = ['q_proj'] + ([] if shared else (['k_proj'] if k_eq_v else ['k_proj', 'v_proj']))
        param = deep_getattr(attn, 'linear_qkv.weight') if attn is not None else None
        qpg = nq // ng
        if to_mcore:
            if param is None:
                return
            parts = [self._load_hf(hf_sd, f'{ap}{n}.weight') for n in names]
            if shared:
                full = parts[0]
            else:
                h = parts[0].shape[1]
                grouped = [parts[0].view(ng, qpg * d, h)] + [p_.view(ng, d, h) for p_ in parts[1:]]
                full = torch.cat(grouped, dim=1).reshape(-1, h)
            self._put(param, full, 0)
            return
        if not self._agree(param is not None, self._device):
            return
        full = self._get(param, 0)
        if full is None:
            return
        if shared:
            self._emit(hf_sd, f'{ap}q_proj.weight', full)
            return
        h = full.shape[1]
        g = full.view(ng, (qpg + len(names) - 1) * d, h)
        self._emit(hf_sd, f'{ap}q_proj.weight', g[:, :qpg * d].reshape(-1, h))
        for j, n in enumerate(names[1:]):
            self._emit(hf_sd, f'{ap}{n}.weight', g[:, (qpg + j) * d:(qpg + j + 1) * d].reshape(-1, h))

    # ------------------------------------------------------------------ LoRA adapters (PEFT format)
    def _qkv_names(self, kind):
        _, _, _, k_eq_v, shared, _ = kind
        return ['q_proj'] + ([] if shared else (['k_proj'] if k_eq_v else ['k_proj', 'v_proj']))

    def _peft_layer_slots(self, layer_idx: int):
        kind = self.kinds[layer_idx]
        slots = [('self_attention.linear_qkv', 'custom_col', 'self_attn.', self._qkv_names(kind)),
                 ('self_attention.linear_proj', 'row', 'self_attn.', ['o_proj']),
                 ('mlp.linear_fc1', 'glu', 'mlp.', ['gate_proj', 'up_proj']),
                 ('mlp.linear_fc2', 'row', 'mlp.', ['down_proj'])]
        if getattr(self.tc, 'hidden_size_per_layer_input', 0):
            slots.append(('per_layer_input_gate', 'column', '', ['per_layer_input_gate']))
            slots.append(('per_layer_projection', 'row', '', ['per_layer_projection']))
        if getattr(self.tc, 'enable_moe_block', False):
            slots.append(('experts_mlp.router', 'replicated', 'router.', ['proj']))
            slots.append(('experts_mlp.experts.linear_fc1', 'grouped_glu', 'experts.', ['gate_proj', 'up_proj']))
            slots.append(('experts_mlp.experts.linear_fc2', 'grouped_row', 'experts.', ['down_proj']))
        return slots

    def _peft_model_slots(self):
        if not getattr(self.tc, 'hidden_size_per_layer_input', 0):
            return None
        return [('per_layer_model_projection', 'column', '', ['per_layer_model_projection'])], self.lm_prefix

    def _kind_of(self, layer_prefix: str):
        return self.kinds[int(layer_prefix.rstrip('.').rsplit('.', 1)[1])]

    def _peft_split(self, layer_prefix: str, path: str, B, names):
        """``lora_B`` of the packed q / k / v projection (rows grouped per KV head) -> one matrix per projection."""
        _, d, ng, _, shared, _ = self._kind_of(layer_prefix)
        if shared:
            return [B]
        qpg, r = self.config.num_attention_heads // ng, B.shape[1]
        g = B.view(ng, (qpg + len(names) - 1) * d, r)
        return [g[:, :qpg * d].reshape(-1, r)] + [g[:, (qpg + j) * d:(qpg + j + 1) * d].reshape(-1, r)
                                                  for j in range(len(names) - 1)]

    def _peft_join(self, layer_prefix: str, path: str, parts, names):
        _, d, ng, _, shared, _ = self._kind_of(layer_prefix)
        if shared:
            return parts[0]
        qpg, r = self.config.num_attention_heads // ng, parts[0].shape[1]
        grouped = [parts[0].view(ng, qpg * d, r)] + [p_.view(ng, d, r) for p_ in parts[1:]]
        return torch.cat(grouped, dim=1).reshape(-1, r)

    def _set_layer_state(self, layer, hf_sd, prefix: str, layer_idx: int, to_mcore: bool):
        kind = self.kinds[layer_idx]
        attn = layer.self_attention if layer is not None else None
        ap = f'{prefix}self_attn.'
        self._set_gemma_qkv(attn, hf_sd, ap, kind, to_mcore)
        self._direct(attn, 'linear_qkv.layer_norm_weight', hf_sd, prefix + 'input_layernorm.weight', to_mcore)
        self._direct(attn, 'q_layernorm.weight', hf_sd, ap + 'q_norm.weight', to_mcore)
        if not kind[4]:
            self._direct(attn, 'k_layernorm.weight', hf_sd, ap + 'k_norm.weight', to_mcore)
        self._direct(attn, 'linear_proj.weight', hf_sd, ap + 'o_proj.weight', to_mcore, tp_dim=1)
        mlp = layer.mlp if layer is not None else None
        self._direct(mlp, 'linear_fc1.layer_norm_weight', hf_sd, prefix + 'pre_feedforward_layernorm.weight', to_mcore)
        self._set_dense_mlp(mlp, hf_sd, prefix + 'mlp.', to_mcore)
        for key in ('post_attention_layernorm', 'post_feedforward_layernorm'):
            self._direct(layer, f'{key}.weight', hf_sd, f'{prefix}{key}.weight', to_mcore)
        if getattr(self.tc, 'hidden_size_per_layer_input', 0):
            self._direct(layer, 'per_layer_input_gate.weight', hf_sd, prefix + 'per_layer_input_gate.weight', to_mcore,
                         tp_dim=0)
            self._direct(layer, 'per_layer_projection.weight', hf_sd, prefix + 'per_layer_projection.weight', to_mcore,
                         tp_dim=1)
            self._direct(layer, 'post_per_layer_input_norm.weight', hf_sd, prefix + 'post_per_layer_input_norm.weight',
                         to_mcore)
        self._direct(layer, 'layer_scalar', hf_sd, prefix + 'layer_scalar', to_mcore, optional=True)
        if getattr(self.tc, 'enable_moe_block', False):
            moe = layer.experts_mlp if layer is not None else None
            self._direct(moe, 'router.weight', hf_sd, prefix + 'router.proj.weight', to_mcore)
            self._direct(moe, 'scale', hf_sd, prefix + 'router.scale', to_mcore)
            self._direct(moe, 'per_expert_scale', hf_sd, prefix + 'router.per_expert_scale', to_mcore)
            self._set_experts(moe.experts if moe is not None else None, hf_sd, prefix, to_mcore)
            self._direct(moe, 'pre_feedforward_layernorm_2.weight', hf_sd,
                         prefix + 'pre_feedforward_layernorm_2.weight', to_mcore)
            for key in ('post_feedforward_layernorm_1', 'post_feedforward_layernorm_2'):
                self._direct(layer, f'{key}.weight', hf_sd, f'{prefix}{key}.weight', to_mcore)

    def _convert_pre_process(self, model, hf_sd, to_mcore: bool):
        super()._convert_pre_process(model, hf_sd, to_mcore)
        if not getattr(self.tc, 'hidden_size_per_layer_input', 0):
            return
        has = model is not None and getattr(model, 'pre_process', False)
        m = model if has else None
        rows_hf = self.tc.vocab_size_per_layer_input
        tab = m.embed_tokens_per_layer if has else None
        rows = tab.num_embeddings if has else rows_hf
        self._direct(tab, 'weight', hf_sd, self.lm_prefix + 'embed_tokens_per_layer.weight', to_mcore, tp_dim=0,
                     to_mg=lambda w: self._pad_vocab(w, rows), to_hf=lambda w: w[:rows_hf])
        self._direct(m, 'per_layer_model_projection.weight', hf_sd,
                     self.lm_prefix + 'per_layer_model_projection.weight', to_mcore, tp_dim=0)
        self._direct(m, 'per_layer_projection_norm.weight', hf_sd,
                     self.lm_prefix + 'per_layer_projection_norm.weight', to_mcore)


# ------------------------------------------------------------------------------------------------- towers
class Gemma4Vit(HuggingFaceVit):
    module_mapping = {'model.vision_tower': 'vision_tower', 'model.embed_vision': 'embed_vision',
                      'model.audio_tower': 'audio_tower', 'model.embed_audio': 'embed_audio'}
    _vision_tower = ['vision_tower', 'audio_tower']
    _aligner = ['embed_vision', 'embed_audio']

    def prepare_model(self, hf_config):
        from transformers import AutoModel
        from transformers.models.gemma4.modeling_gemma4 import Gemma4MultimodalEmbedder
        self.vision_tower = AutoModel.from_config(hf_config.vision_config)
        dtype = next(self.vision_tower.parameters()).dtype
        has_audio = getattr(hf_config, 'audio_config', None) is not None
        self.audio_tower = AutoModel.from_config(hf_config.audio_config) if has_audio else None
        self.embed_vision = Gemma4MultimodalEmbedder(hf_config.vision_config, hf_config.text_config).to(dtype)
        self.embed_audio = Gemma4MultimodalEmbedder(hf_config.audio_config, hf_config.text_config).to(dtype) \
            if has_audio else None
        self.prepare_language_model(hf_config)

    def prepare_language_model(self, hf_config):
        self.embed_scale = float(text_config_of(self.config).hidden_size) ** 0.5

    def get_inputs_embeds_language_model(self, inputs_embeds, **inputs):
        scaled = inputs_embeds * torch.tensor(self.embed_scale, dtype=inputs_embeds.dtype)
        return {'inputs_embeds': scaled, 'llm_input_ids': inputs.get('input_ids')}

    def _vision(self, pixel_values, position_ids):
        """Soft tokens of the valid patches of every image, projected into the language model's width."""
        p = next(self.vision_tower.parameters())
        out = self.vision_tower(pixel_values=pixel_values.to(device=p.device, dtype=p.dtype),
                                pixel_position_ids=position_ids.to(p.device))
        return self.embed_vision(inputs_embeds=out.last_hidden_state)

    def _put_features(self, embeds, mask, feats):
        if feats is None:
            return embeds
        feats = feats.to(device=embeds.device, dtype=embeds.dtype)
        return embeds.masked_scatter(mask.unsqueeze(-1).expand_as(embeds).to(embeds.device), feats)

    def get_inputs_embeds(self, inputs_embeds, **inputs):
        cfg = self.hf_config
        res = self.get_inputs_embeds_language_model(inputs_embeds, **inputs)
        ids = inputs['input_ids']
        masks = {k: ids == getattr(cfg, f'{k}_token_id', -1) for k in ('image', 'video', 'audio')}
        llm_ids = ids.clone()
        llm_ids[masks['image'] | masks['video'] | masks['audio']] = cfg.text_config.pad_token_id or 0
        e = res['inputs_embeds']
        if inputs.get('pixel_values') is not None:
            e = self._put_features(e, masks['image'],
                                   self._vision(inputs['pixel_values'], inputs.get('image_position_ids')))
        if inputs.get('pixel_values_videos') is not None:       # [videos, frames, patches, ...]: frames are images
            e = self._put_features(e, masks['video'], self._vision(inputs['pixel_values_videos'].flatten(0, 1),
                                                                   inputs['video_position_ids'].flatten(0, 1)))
        if inputs.get('input_features') is not None and inputs.get('input_features_mask') is not None \
                and self.audio_tower is not None:
            out = self.audio_tower(inputs['input_features'], inputs['input_features_mask'], return_dict=True)
            feats = self.embed_audio(inputs_embeds=out.last_hidden_state)
            e = self._put_features(e, masks['audio'], feats[out.attention_mask])
        return {'inputs_embeds': e, 'llm_input_ids': llm_ids}


class _Gemma4TextLoader(ModelLoader):
    model_cls = Gemma4TextModel


class _Gemma4Loader(ModelLoader):

    def get_model_cls(self):
        return Gemma4TextModel if self.config.language_model_only and not self.config.is_multimodal else Gemma4Model


register_model(ModelMeta(ModelType.gemma4, ['gemma4'], bridge_cls=Gemma4Bridge, visual_cls=Gemma4Vit,
                         loader=_Gemma4Loader))
register_model(ModelMeta(ModelType.gemma4_unified, ['gemma4_unified'], bridge_cls=Gemma4Bridge, visual_cls=Gemma4Vit,
                         loader=_Gemma4Loader))
register_model(ModelMeta('gemma4_text', ['gemma4_text'], bridge_cls=Gemma4Bridge, loader=_Gemma4TextLoader))
