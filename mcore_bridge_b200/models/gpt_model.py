"""``GPTModel``: embedding -> decoder stack -> (MTP) -> output head / loss, for one pipeline stage.

Public ``forward`` signature follows the reference model (``src/mcore_bridge/model/gpt_model.py:246-260``):
``input_ids [b, s]``, ``position_ids``, ``attention_mask``, ``labels`` ... and returns either logits
``[b, s, V/tp]`` or, when ``labels`` are given, the per-token loss ``[b, s]`` (the caller masks and
averages).  Internally activations are token-major ``[T, H]`` with ``T = b*s``; sequences of a packed
batch are delimited by ``packed_seq_params.cu_seqlens_q``; under sequence parallelism the stack works on
``[T/tp, H]`` shards, under context parallelism on the zig-zag chunks the caller already selected with
``split_cp_inputs``.

Task heads: ``causal_lm`` (vocab-parallel head, fused linear + cross-entropy), ``seq_cls`` (replicated
``num_labels`` head), ``embedding`` (L2-normalised hidden state, no head) and ``generative_reranker``
(logit difference of two vocabulary rows).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch
from torch import nn

from ..layers.context import ForwardContext, PackedSeqParams
from ..layers.embedding import LanguageModelEmbedding
from ..layers.linear import ColumnParallelLinear, ReplicatedLinear
from ..ops.cross_entropy import fused_linear_cross_entropy, vocab_parallel_cross_entropy
from ..ops.linear import LinearSpec, linear
from ..parallel import mappings as M
from ..parallel import state as ps
from ..utils.logger import get_logger
from .rope import RotaryEmbedding
from .transformer_block import TransformerBlock

logger = get_logger()


def padded_vocab(vocab_size: int, tp: int) -> int:
    """Vocabulary rounded up to a multiple of TP (reference ``src/mcore_bridge/model/gpt_model.py:70-71``)."""
    return (vocab_size + tp - 1) // tp * tp


class GPTModel(nn.Module):
    # names of extra keyword inputs a multimodal wrapper forwards to the decoder blocks untouched
    extra_forward_keys = []
    block_cls = TransformerBlock          # families with their own decoder stack replace this

    def __init__(self, config, pre_process: bool = True, post_process: bool = True, vp_stage: Optional[int] = None):
        super().__init__()
        self.config = config
        self.pre_process, self.post_process, self.vp_stage = pre_process, post_process, vp_stage
        tp = ps.get_world_size('tp')
        self.vocab_size = padded_vocab(config.padded_vocab_size, tp)
        self.share_embeddings_and_output_weights = not config.untie_embeddings_and_output_weights
        if pre_process or (config.mtp_num_layers and post_process):
            self.embedding = LanguageModelEmbedding(config, self.vocab_size)
        else:
            self.embedding = None
        if config.position_embedding_type in ('rope', 'mrope'):
            self.rotary_pos_emb = RotaryEmbedding(config)
        else:
            self.rotary_pos_emb = None
        self.decoder = self.block_cls(config, pre_process, post_process, vp_stage)
        self.mtp = None
        if post_process and config.mtp_num_layers:
            from ..layers.mtp import MultiTokenPredictionBlock
            self.mtp = MultiTokenPredictionBlock(config)
        self.output_layer = None
        if post_process:
            task = config.task_type
            if task == 'causal_lm' or task == 'generative_reranker':
                self.output_layer = ColumnParallelLinear(config.hidden_size, self.vocab_size, config, bias=False,
                                                         sequence_parallel=False, fp8=False)
                extra = int(config.mtp_unroll_steps or config.mtp_num_layers or 0) if self.mtp is not None else 0
                # the last pipeline stage of a model with MTP holds an embedding of its own (the MTP depths look their
                # tokens up): with tied weights it is the head's matrix there too
                tie_here = self.share_embeddings_and_output_weights and self.embedding is not None
                if tie_here:
                    self.output_layer.weight = self.embedding.word_embeddings.weight
                    # embedding lookup and head (and, per MTP depth, one more of each) produce a gradient for this
                    # tensor in every backward pass; the bucket waits for all of them
                    self.output_layer.weight.grad_contributions = (1 if pre_process else 0) + 1 + 2 * extra
                elif self.mtp is not None:
                    # untied, with MTP: every depth looks up the embedding and applies the head once more
                    self.output_layer.weight.grad_contributions = 1 + extra
                    if self.embedding is not None:
                        self.embedding.word_embeddings.weight.grad_contributions = (1 if pre_process else 0) + extra
            elif task == 'seq_cls':
                self.output_layer = ReplicatedLinear(config.hidden_size, config.num_labels, config, bias=False,
                                                     sequence_parallel_grad=False)
        if ps.get_pipeline_model_parallel_world_size() > 1:
            lm_head = post_process and self.output_layer is not None and \
                config.task_type in ('causal_lm', 'generative_reranker')
            if self.share_embeddings_and_output_weights:
                # the stages at the two ends of the pipeline each hold a copy of the tied matrix
                if pre_process and self.embedding is not None:
                    self.embedding.word_embeddings.weight.shared_embedding = True
                if post_process and not pre_process and lm_head:
                    self.output_layer.weight.shared_embedding = True
            elif config.mtp_num_layers and self.embedding is not None and (pre_process or post_process):
                # untied, with MTP: the embedding exists on the first stage and, for the MTP depths, on the last one;
                # the two copies sum their gradients like a tied pair
                self.embedding.word_embeddings.weight.shared_embedding = True
        self._extra_tables: Dict[str, RotaryEmbedding] = {}

    # ------------------------------------------------------------------ pipeline plumbing
    def set_input_tensor(self, input_tensor):
        if isinstance(input_tensor, (list, tuple)):
            input_tensor = input_tensor[0]
        self.decoder.set_input_tensor(input_tensor)

    def get_input_tensor(self):
        return self.decoder.input_tensor

    def shared_embedding_or_output_weight(self):
        if self.pre_process:
            return self.embedding.word_embeddings.weight
        if self.post_process and self.output_layer is not None:
            return self.output_layer.weight
        return None

    # ------------------------------------------------------------------ context construction
    def build_context(self, input_ids: Optional[torch.Tensor], position_ids: Optional[torch.Tensor],
                      attention_mask: Optional[torch.Tensor], packed_seq_params: Optional[PackedSeqParams],
                      batch: int, seq: int, device) -> ForwardContext:
        cfg = self.config
        cp = ps.get_world_size('cp')
        T = batch * seq
        if packed_seq_params is not None and packed_seq_params.cu_seqlens_q is not None:
            src = packed_seq_params.cu_seqlens_q
            cu = src.to(device=device, dtype=torch.int32)
            if cu is not src:
                # keep the boundaries readable on the host: from the caller's host copy if it is one, else from the
                # values a previous copy already carries
                if src.device.type == 'cpu':
                    from ..utils.torch_utils import attach_host_list
                    attach_host_list(cu, src)
                elif getattr(src, '_host_list', None) is not None:
                    cu._host_list = src._host_list
            max_len = packed_seq_params.max_seqlen_q
        else:
            cu = torch.arange(0, (batch + 1) * seq * cp, seq * cp, dtype=torch.int32, device=device)
            max_len = seq * cp
        if position_ids is None:
            if cp > 1:
                raise ValueError('position_ids are required under context parallelism')
            starts = cu[:-1].to(torch.int64)
            seg = torch.searchsorted(cu[1:].to(torch.int64).contiguous(), torch.arange(T, device=device), right=True)
            position_ids = torch.arange(T, device=device) - starts[seg]
        if position_ids.dim() == 3:        # mrope [3, b, s]
            pos = position_ids.reshape(3, -1)
        else:
            pos = position_ids.reshape(-1)
        ctx = ForwardContext(cu_seqlens=cu, max_seqlen=max_len, position_ids=pos, input_ids=input_ids)
        if device.type == 'cuda' and cp == 1:
            from ..ops.attention_cuda import seq_start_from_cu
            ctx.seq_start = seq_start_from_cu(cu, T, device)
        if self.rotary_pos_emb is not None:
            seq_len_hint = int(max_len) if max_len is not None else None
            ctx.cos, ctx.sin = self.rotary_pos_emb(pos.to(device), seq_len_hint)
        for key, emb in self._extra_tables.items():
            ctx.rope_tables[key] = emb(pos.to(device))
        if attention_mask is not None and attention_mask.dim() == 2:
            full_pad = ~attention_mask.reshape(-1).bool()          # [T] True where padding
            ctx.extra['full_padding_mask'] = full_pad
            ctx.padding_mask = M.split_dim0(full_pad, 'tp') if (cfg.sequence_parallel and
                                                                ps.get_world_size('tp') > 1) else full_pad
        if cfg.moe_router_load_balancing_type == 'seq_aux_loss' and cfg.num_moe_experts:
            if cp == 1:
                seg = torch.searchsorted(cu[1:].to(torch.int64).contiguous(), torch.arange(T, device=device),
                                         right=True)
            else:  # per-sequence chunks of equal share: token i of this rank's stream belongs to seq by scaled cu
                seg = torch.searchsorted((cu[1:].to(torch.int64) // cp).contiguous(),
                                         torch.arange(T, device=device), right=True)
            ctx.num_seqs = cu.numel() - 1
            ctx.seg_ids = M.split_dim0(seg, 'tp') if (cfg.sequence_parallel and ps.get_world_size('tp') > 1) else seg
        return ctx

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None,
                attention_mask: Optional[torch.Tensor] = None, decoder_input: Optional[torch.Tensor] = None,
                labels: Optional[torch.Tensor] = None, inference_context=None,
                packed_seq_params: Optional[PackedSeqParams] = None, extra_block_kwargs: Optional[dict] = None,
                runtime_gather_output: Optional[bool] = None, loss_mask: Optional[torch.Tensor] = None,
                **kwargs):
        cfg = self.config
        sp = cfg.sequence_parallel and ps.get_world_size('tp') > 1
        if input_ids is not None:
            batch, seq = (input_ids.shape if input_ids.dim() == 2 else (1, input_ids.shape[0]))
            device = input_ids.device
        elif decoder_input is not None:
            batch, seq = decoder_input.shape[0], decoder_input.shape[1]
            device = decoder_input.device
        else:
            ref = labels if labels is not None else position_ids
            batch, seq = ref.shape[-2], ref.shape[-1]
            device = ref.device
        ctx = self.build_context(input_ids, position_ids, attention_mask, packed_seq_params, batch, seq, device)
        if extra_block_kwargs:
            ctx.extra.update(extra_block_kwargs)
        hidden = None
        if self.pre_process:
            if decoder_input is not None:
                hidden = self.on_decoder_input(decoder_input.reshape(batch * seq, -1), ctx)
                if sp:
                    hidden = M.scatter_to_sequence_parallel_region(hidden)
            else:
                hidden = self.embed(input_ids.reshape(-1), ctx, sp)
        out = self.decoder(hidden, ctx)
        taps = None
        if isinstance(out, tuple):
            out, taps = out
        if not self.post_process:
            return out
        result = self._postprocess(out, ctx, input_ids, labels, loss_mask, batch, seq, sp, runtime_gather_output)
        if taps is not None:
            return result, taps
        return result

    def on_decoder_input(self, hidden_full: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        """Hook for embeddings computed by the caller (multimodal wrappers): sees the full token stream ``[T, H]``
        before the sequence-parallel scatter."""
        return hidden_full

    def finalize_logits(self, logits: torch.Tensor) -> torch.Tensor:
        """Hook applied to the (vocab-parallel) logits before they are returned."""
        return logits

    def embed(self, flat_ids: torch.Tensor, ctx: ForwardContext, sp: bool) -> torch.Tensor:
        return self.embedding(flat_ids.clamp(min=0), scatter_to_sequence_parallel=sp)

    # ------------------------------------------------------------------ heads
    def _head_weight(self):
        if self.share_embeddings_and_output_weights:
            w = self.shared_embedding_or_output_weight()
            if w is not None:
                return w
        return self.output_layer.weight

    def _lm_loss(self, hidden_full: torch.Tensor, labels_flat: torch.Tensor) -> torch.Tensor:
        """``hidden_full [T, H]`` already gathered over SP and registered for TP gradient reduction."""
        cfg = self.config
        w = self._head_weight()
        if cfg.cross_entropy_loss_fusion:
            return fused_linear_cross_entropy(hidden_full, w, labels_flat, 'tp')
        logits = linear(hidden_full, w, None, LinearSpec())
        return vocab_parallel_cross_entropy(logits.float(), labels_flat, 'tp')

    def _gather_for_head(self, hidden: torch.Tensor, sp: bool) -> torch.Tensor:
        if sp:
            return M.gather_from_sequence_parallel_region(hidden, 'tp', tensor_parallel_output_grad=True)
        return M.copy_to_tensor_model_parallel_region(hidden, 'tp')

    def _postprocess(self, hidden, ctx, input_ids, labels, loss_mask, batch, seq, sp, runtime_gather_output):
        cfg = self.config
        task = cfg.task_type
        if self.mtp is not None and labels is not None and self.training:
            hidden = self.mtp.forward_with_loss(self, hidden, ctx, input_ids, labels, loss_mask, batch, seq, sp)
        if task == 'embedding':
            h = M.gather_from_sequence_parallel_region(hidden, 'tp', False) if sp else hidden
            h = torch.nn.functional.normalize(h.float(), p=2, dim=-1).to(hidden.dtype)
            return h.view(batch, seq, -1)
        if task == 'seq_cls':
            h = M.gather_from_sequence_parallel_region(hidden, 'tp', False) if sp else hidden
            return self.output_layer(h).view(batch, seq, -1)
        if task == 'generative_reranker':
            return self._reranker(hidden, batch, seq, sp)
        h = self._gather_for_head(hidden, sp)
        if labels is None:
            logits = self.finalize_logits(linear(h, self._head_weight(), None, LinearSpec()))
            if runtime_gather_output:
                logits = M.gather_from_tensor_model_parallel_region(logits, 'tp')
            return logits.view(batch, seq, -1)
        loss = self._lm_loss(h, labels.reshape(-1))
        return loss.view(batch, seq)

    def _reranker(self, hidden, batch, seq, sp):
        """Score = logit(positive token) - logit(negative token); only two vocabulary rows are used, each
        living on one TP rank, so the other ranks contribute zero and the result is all-reduced (reference
        ``src/mcore_bridge/model/gpt_model.py:356-416``)."""
        pos_id = int(os.environ.get('GENERATIVE_RERANKER_POSITIVE_TOKEN_ID', os.environ.get(
            'GENERATIVE_RERANKER_POSITIVE_TOKEN', '9693')))
        neg_id = int(os.environ.get('GENERATIVE_RERANKER_NEGATIVE_TOKEN_ID', os.environ.get(
            'GENERATIVE_RERANKER_NEGATIVE_TOKEN', '2152')))
        h = self._gather_for_head(hidden, sp)
        w = self._head_weight()
        vl = w.shape[0]
        start = ps.get_rank_in('tp') * vl if ps.get_world_size('tp') > 1 else 0
        rows = []
        for tid in (pos_id, neg_id):
            loc = tid - start
            if 0 <= loc < vl:
                rows.append(w[loc])
            else:
                rows.append(torch.zeros_like(w[0]))
        w2 = torch.stack(rows)
        logits = torch.nn.functional.linear(h, w2)                  # [T, 2]
        logits = M.reduce_from_tensor_model_parallel_region(logits, 'tp')
        return (logits[:, 0] - logits[:, 1]).view(batch, seq, 1)
