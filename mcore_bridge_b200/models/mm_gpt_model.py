"""Language model + media towers.

``MultimodalGPTModel`` owns a ``language_model`` (the native ``GPTModel``) and, on the first pipeline stage, a
``visual`` tower wrapper.  Its forward embeds the *full* token stream without sequence-parallel scattering, lets the
tower write media embeddings into the placeholder rows, then hands the result to the language model as
``decoder_input`` — the language model applies the CP split and SP scatter exactly as it does for text.  Extra
outputs of the tower (deepstack features and the like) travel in ``extra_block_kwargs``.

Parity: reference ``src/mcore_bridge/model/mm_gpt_model.py:16-122`` (which reaches the same result by temporarily
replacing the embedding class's forward).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..layers.context import PackedSeqParams
from ..utils.megatron_utils import reconstruct_tensor_cp, split_cp_inputs
from .gpt_model import GPTModel


class MultimodalGPTModel(nn.Module):
    language_model_cls = GPTModel

    def __init__(self, config, pre_process: bool = True, post_process: bool = True, vp_stage: Optional[int] = None,
                 **kwargs):
        super().__init__()
        self.config = config
        self.pre_process, self.post_process, self.vp_stage = pre_process, post_process, vp_stage
        self.language_model = self.language_model_cls(config, pre_process=pre_process, post_process=post_process,
                                                      vp_stage=vp_stage, **kwargs)
        self.share_embeddings_and_output_weights = self.language_model.share_embeddings_and_output_weights
        self.model_meta = config.model_meta
        self.visual = None
        if pre_process and self.model_meta.visual_cls is not None:
            self.visual = self.model_meta.visual_cls(config)

    # the trainer and the bridge address the decoder through these
    @property
    def decoder(self):
        return self.language_model.decoder

    @property
    def embedding(self):
        return self.language_model.embedding

    @property
    def output_layer(self):
        return self.language_model.output_layer

    @property
    def mtp(self):
        return self.language_model.mtp

    def embed_full_stream(self, input_ids: torch.Tensor, packed_seq_params, media: dict):
        """Text embeddings of the full stream ``[b, s, H]`` with media written in; returns (embeds, extras)."""
        lm = self.language_model
        emb = lm.embedding(input_ids.clamp(min=0), scatter_to_sequence_parallel=False)
        extras = {}
        if self.visual is not None:
            inputs = dict(media)
            inputs.update(input_ids=input_ids, packed_seq_params=packed_seq_params)
            fn = (self.visual.get_inputs_embeds_language_model if self.config.language_model_only
                  else self.visual.get_inputs_embeds)
            res = fn(emb, **inputs)
            if isinstance(res, dict):
                emb = res.pop('inputs_embeds')
                extras = res
            else:
                emb = res
        return emb, extras

    def forward(self, input_ids: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None,
                attention_mask: Optional[torch.Tensor] = None, decoder_input: Optional[torch.Tensor] = None,
                labels: Optional[torch.Tensor] = None, inference_context=None,
                packed_seq_params: Optional[PackedSeqParams] = None, **kwargs):
        cfg = self.config
        lm = self.language_model
        cp = cfg.context_parallel_size
        cu = getattr(packed_seq_params, 'cu_seqlens_q', None)
        passthrough = {k: kwargs.pop(k) for k in list(kwargs) if k in lm.extra_forward_keys}
        loss_mask = kwargs.pop('loss_mask', None)
        runtime_gather_output = kwargs.pop('runtime_gather_output', None)
        # callers may pass the full ids with already-split position ids, or ids that are already split
        ids_are_full = cp > 1 and input_ids is not None and position_ids is not None and \
            position_ids.shape[-1] * cp == input_ids.shape[-1]
        extras = {}
        if decoder_input is None and self.pre_process and input_ids is not None:
            full_ids = input_ids if (cp == 1 or ids_are_full) else \
                reconstruct_tensor_cp(input_ids, packed_seq_params, 1)
            decoder_input, extras = self.embed_full_stream(full_ids, packed_seq_params, kwargs)
            if cp > 1:
                decoder_input = split_cp_inputs(decoder_input, cu, 1)
        if ids_are_full:
            input_ids = split_cp_inputs(input_ids, cu, 1)
        extras.update(passthrough)
        return lm(input_ids=input_ids, position_ids=position_ids, attention_mask=attention_mask,
                  decoder_input=decoder_input, labels=labels, inference_context=inference_context,
                  packed_seq_params=packed_seq_params, extra_block_kwargs=extras, loss_mask=loss_mask,
                  runtime_gather_output=runtime_gather_output)

    def set_input_tensor(self, t):
        return self.language_model.set_input_tensor(t)

    def get_input_tensor(self):
        return self.language_model.get_input_tensor()

    def shared_embedding_or_output_weight(self):
        return self.language_model.shared_embedding_or_output_weight()
