"""``ModelConfig``: every architecture / parallelism / precision knob of a model, as one dataclass.

Field names follow the reference's ``ModelConfig`` (``src/mcore_bridge/config/model_config.py:115-245``)
and the Megatron ``TransformerConfig`` fields it inherits, because ``hf_to_mcore_config`` produces
exactly those keys and user scripts pass them by name.  Here it is a standalone dataclass: there is
no Megatron base class.
"""
from __future__ import annotations

import copy
import re
from dataclasses import dataclass
from typing import Any, Callable, List, Literal, Optional, Tuple, Union

import torch
import torch.nn.functional as F

from ..utils.logger import get_logger
from ..utils.utils import json_parse_to_dict

logger = get_logger()

_PATTERN_OK = re.compile(r'^[,\d\[\]\(\)\+\*\s]*$')


def _eval_pattern(pattern: str) -> List[int]:
    """Evaluates the small list language used for layer patterns, e.g. ``"([0]*3+[1])*2"``."""
    if not isinstance(pattern, str) or not _PATTERN_OK.match(pattern):
        raise ValueError(f'Invalid pattern: {pattern}')
    return list(eval(pattern, {'__builtins__': {}}, {}))  # only digits, brackets, + and * pass the regex


def _int_or_pattern(x):
    if x is None or isinstance(x, (int, list, tuple)):
        return x
    assert isinstance(x, str)
    return _eval_pattern(x) if '[' in x else int(x)


no_rope_freq_type = _int_or_pattern
linear_attn_freq_type = _int_or_pattern
moe_freq_type = _int_or_pattern


def tuple_type(x):
    """``"1,2"`` / ``"(1,2)"`` -> ``(1, 2)``."""
    if x is None or isinstance(x, tuple):
        return x
    if isinstance(x, list):
        return tuple(x)
    return tuple(int(i) for i in x.strip('()').split(','))


def quick_gelu(x):
    return x * torch.sigmoid(1.702 * x)


@dataclass
class ModelConfig:
    mcore_model_type: Optional[str] = None  # inferred from hf_model_type
    hf_model_type: Optional[str] = None
    llm_model_type: Optional[str] = None
    padded_vocab_size: Optional[int] = None
    rope_scaling: Optional[Union[dict, str]] = None
    attention_scaling: float = 1.

    # model
    num_layers: Optional[int] = None
    hidden_size: Optional[int] = None
    ffn_hidden_size: Optional[int] = None
    num_attention_heads: Optional[int] = None
    num_query_groups: Optional[int] = None
    softmax_type: Literal['vanilla', 'off-by-one', 'learnable'] = 'vanilla'
    softmax_scale: Optional[float] = None
    window_size: Optional[Union[str, Tuple[int, int]]] = None
    window_attn_skip_freq: Optional[Union[str, int, List[int]]] = None
    max_position_embeddings: Optional[int] = None

    position_embedding_type: Literal['learned_absolute', 'rope', 'mrope', 'none'] = 'rope'
    rotary_base: int = 10000
    rotary_percent: float = 1.
    rotary_interleaved: bool = False
    original_max_position_embeddings: Optional[int] = None
    partial_rotary_factor: Optional[float] = None
    mrope_section: Optional[List[int]] = None
    mrope_interleaved: bool = False

    normalization: Literal['LayerNorm', 'RMSNorm'] = 'RMSNorm'
    layernorm_epsilon: float = 1e-5
    swiglu: bool = True
    quick_geglu: bool = False
    gated_linear_unit: bool = False
    activation_func: Optional[Callable] = None
    activation_func_clamp_value: Optional[float] = None
    glu_linear_offset: float = 0.
    untie_embeddings_and_output_weights: bool = True
    add_bias_linear: bool = False
    add_qkv_bias: bool = True
    attention_dropout: float = 0.
    hidden_dropout: float = 0.
    kv_channels: Optional[int] = None
    qk_layernorm: bool = False
    qk_l2_norm: bool = False
    # single-rank dense path: recompute norm / gated activation in backward instead of storing them
    lean_activations: bool = True
    qk_layernorm_full: bool = False          # q/k RMSNorm over all heads' channels at once (OLMoE, MiniMax-M2)
    post_sublayer_layernorm: bool = False    # sandwich norms after attention and MLP outputs (GLM-4)
    no_rope_freq: Optional[Union[int, str, List[int]]] = None
    moe_apply_probs_on_input: Optional[bool] = None
    bias_dropout_fusion: bool = True

    # moe
    num_moe_experts: Optional[int] = None
    moe_layer_freq: Union[str, int, List[int]] = '1'
    moe_ffn_hidden_size: Optional[int] = None
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_router_topk: int = 2
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_router_pre_softmax: bool = False
    moe_router_score_function: Literal['sigmoid', 'softmax'] = 'softmax'
    moe_router_bias_update_rate: float = 1e-3
    moe_router_enable_expert_bias: bool = False
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_load_balancing_type: Literal['aux_loss', 'seq_aux_loss', 'global_aux_loss', 'sinkhorn',
                                            'none'] = 'aux_loss'
    moe_aux_loss_coeff: float = 0.
    moe_z_loss_coeff: Optional[float] = None
    moe_shared_expert_gate: bool = False
    moe_expert_capacity_factor: Optional[float] = None
    moe_permute_fusion: bool = True

    # mla
    multi_latent_attention: bool = False
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 32
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 128
    mla_rope_interleaved: Optional[bool] = None  # None -> True (DeepSeek); GLM-5 checkpoints use rotate-half

    # qwen3_next / qwen3_5
    linear_attention_freq: Optional[Union[str, int, List[int]]] = None
    linear_num_key_heads: Optional[int] = None
    linear_num_value_heads: Optional[int] = None
    linear_key_head_dim: Optional[int] = None
    linear_value_head_dim: Optional[int] = None
    linear_conv_kernel_dim: Optional[int] = None
    layernorm_zero_centered_gamma: bool = False
    attention_output_gate: bool = False
    linear_decoupled_in_proj: bool = False

    # dsa
    experimental_attention_variant: Optional[Literal['gated_delta_net', 'dsa', 'dsv4_hybrid', 'lightning']] = None
    dsa_indexer_n_heads: Optional[int] = None
    dsa_indexer_head_dim: Optional[int] = None
    dsa_indexer_topk: Optional[int] = None
    dsa_indexer_loss_coeff: float = 0.
    dsa_indexer_use_sparse_loss: bool = False
    dsa_indexer_rotary_interleaved: bool = False

    # deepseek-v4
    csa_window_size: int = 128
    csa_compress_ratios: Optional[List[int]] = None
    csa_compress_rotary_base: float = 40000.0
    o_groups: int = 8
    o_lora_rank: int = 1024
    enable_hyper_connections: bool = False
    num_residual_streams: int = 4
    mhc_sinkhorn_iterations: int = 20
    mhc_init_gating_factor: float = 0.01
    moe_n_hash_layers: int = 0

    # mtp
    mtp_num_layers: Optional[int] = None
    mtp_loss_scaling_factor: float = 0.1
    mtp_decoder_input_detach: bool = False
    mtp_shared_weights: bool = False

    # visual
    language_model_only: bool = False
    hf_config: Optional[Any] = None
    vit_attn_impl: Optional[str] = None

    # parallelism
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    sequence_parallel: bool = False
    num_layers_in_first_pipeline_stage: Optional[int] = None
    num_layers_in_last_pipeline_stage: Optional[int] = None
    account_for_embedding_in_pipeline_split: bool = False
    account_for_loss_in_pipeline_split: bool = False

    # precision
    params_dtype: torch.dtype = torch.float32
    bf16: bool = False
    fp16: bool = False
    pipeline_dtype: Optional[torch.dtype] = None
    fp8: Optional[str] = None  # None | 'e4m3' | 'hybrid'
    # 'blockwise' (128x128 weights, 1x128 activations) | 'delayed' | 'tensorwise' | 'mxfp8'
    fp8_recipe: Optional[str] = None
    fp8_param: bool = False
    fp4: Optional[str] = None
    attention_softmax_in_fp32: bool = True
    cross_entropy_loss_fusion: bool = True
    deterministic_mode: bool = False
    test_mode: bool = False

    # recompute / offload
    recompute_granularity: Optional[Literal['full', 'selective']] = None
    recompute_method: Optional[Literal['uniform', 'block']] = None
    recompute_num_layers: Optional[int] = None
    recompute_modules: Optional[List[str]] = None
    cpu_offloading: bool = False                      # saved activations of the first layers live in pinned host memory
    cpu_offloading_num_layers: Optional[int] = None   # how many leading layers of a stage offload (default: all)
    fine_grained_activation_offloading: bool = False  # offload the saved tensors of the sub-blocks in offload_modules
    # attn_norm / core_attn / attn_proj / mlp_norm / moe_act / expert_fc1 ...
    offload_modules: Optional[List[str]] = None

    # initialisation
    perform_initialization: bool = False
    init_method_std: float = 0.02
    apply_query_key_layer_scaling: Optional[bool] = None
    moe_router_dtype: Optional[Literal['none', 'fp32', 'fp64']] = 'fp32'
    moe_token_dispatcher_type: Literal['allgather', 'alltoall', 'flex'] = 'alltoall'
    moe_grouped_gemm: bool = True
    variable_seq_lengths: bool = True
    calculate_per_token_loss: bool = False

    overlap_p2p_comm: bool = True
    batch_p2p_comm: bool = False
    persist_layer_norm: bool = True
    deallocate_pipeline_outputs: bool = True
    cp_comm_type: Union[str, List[str]] = 'p2p'

    # other
    task_type: Literal['causal_lm', 'seq_cls', 'embedding', 'generative_reranker'] = 'causal_lm'
    num_labels: Optional[int] = None
    mlp_padding_free: bool = False
    extract_layer_indices: Optional[List[int]] = None

    def __post_init__(self):
        from ..models.register import get_mcore_model_type, get_model_meta
        from ..parallel import state as ps
        self._format_config()
        # options that exist in the reference's config but have no implementation here are refused instead of being
        # silently ignored
        if any(self.csa_compress_ratios or []):
            raise NotImplementedError(
                'compressed attention layers (non-zero csa_compress_ratios: the compressed-sparse and heavily-'
                'compressed layers of DeepSeek-V4) are not implemented: the reference takes their core attention from '
                'a '
                'Megatron-Core development branch that is not part of its own source tree.  Sliding-window layers '
                '(ratio 0), hyper-connections and hash-routed MoE layers of the family are available.')
        if self.experimental_attention_variant == 'dsv4_hybrid' and self.mtp_num_layers:
            raise NotImplementedError('DeepSeek-V4: multi-token-prediction layers over hyper-connection streams are '
                                      'not implemented; build the model with mtp_num_layers=None')
        if self.fp8_param:
            # weights stay bf16 views of the optimizer's flat buffers; their fp8 copies (and transposes) are cached and
            # re-quantised only when an optimizer step changes the weight (ops/fp8.py: quantized_weight), which gives
            # fp8_param's run-time effect (no per-micro-batch weight quantisation) but not its memory saving
            from ..utils.logger import get_logger
            get_logger().warning_once('fp8_param: parameters are kept in bf16 with cached fp8 copies; the memory '
                                      'saving of fp8-only parameters is not implemented')
        if isinstance(self.moe_router_dtype, str) and self.moe_router_dtype.lower() == 'none':
            self.moe_router_dtype = None
        if self.moe_shared_expert_intermediate_size == 0:
            self.moe_shared_expert_intermediate_size = None
        if self.num_moe_experts is not None and self.moe_ffn_hidden_size is None:
            self.moe_ffn_hidden_size = self.ffn_hidden_size
        if self.rope_scaling is not None:
            self.rope_scaling = json_parse_to_dict(self.rope_scaling)
            if 'type' in self.rope_scaling and 'rope_type' not in self.rope_scaling:
                self.rope_scaling['rope_type'] = self.rope_scaling['type']
        if self.add_bias_linear:
            self.add_qkv_bias = True
        self.actual_vocab_size = self.padded_vocab_size
        if self.overlap_p2p_comm:
            self.batch_p2p_comm = False
        if self.quick_geglu:
            assert not self.swiglu, 'quick_geglu and swiglu are exclusive'
            self.gated_linear_unit = True
            self.activation_func = quick_gelu
        elif self.swiglu:
            self.activation_func = F.silu
            self.gated_linear_unit = True
        elif self.activation_func is None:
            self.activation_func = F.gelu
        if self.bf16:
            self.params_dtype = torch.bfloat16
        elif self.fp16:
            self.params_dtype = torch.float16
        if self.pipeline_dtype is None:
            self.pipeline_dtype = self.params_dtype
        if self.apply_query_key_layer_scaling is None:
            self.apply_query_key_layer_scaling = self.fp16
        if self.mtp_shared_weights:
            assert self.mtp_num_layers is not None
            self.mtp_unroll_steps = self.mtp_num_layers
            self.mtp_num_layers = 1
        else:
            self.mtp_unroll_steps = self.mtp_num_layers
        if self.csa_compress_ratios is not None and self.mtp_num_layers is not None:
            self.csa_compress_ratios = list(self.csa_compress_ratios) + [0] * self.mtp_num_layers
        if self.mla_rope_interleaved is None:
            self.mla_rope_interleaved = True
        if self.multi_latent_attention:
            # MLA always rotates interleaved pairs of the rope sub-dimension; the flag only applies to the
            # (non-MLA) indexer, see dsa_indexer_rotary_interleaved
            self.rotary_interleaved = False
        if self.kv_channels is None and self.hidden_size and self.num_attention_heads:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.ffn_hidden_size is None and self.hidden_size is not None and self.num_moe_experts is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.expert_tensor_parallel_size is None:
            self.expert_tensor_parallel_size = self.tensor_model_parallel_size
        if self.sequence_parallel and self.tensor_model_parallel_size == 1:
            self.sequence_parallel = False
        if self.recompute_granularity == 'selective' and self.recompute_modules is None:
            self.recompute_modules = ['core_attn']
        if ps.model_parallel_is_initialized():
            st = ps.get_state()
            for cfg_name, have in (('tensor_model_parallel_size', st.tp), ('pipeline_model_parallel_size', st.pp),
                                   ('context_parallel_size', st.cp), ('expert_model_parallel_size', st.ep)):
                if getattr(self, cfg_name) != have:
                    raise ValueError(f'{cfg_name}={getattr(self, cfg_name)} but the process groups were built with '
                                     f'{have}')
        self._validate()
        if self.mcore_model_type is None:
            self.mcore_model_type = get_mcore_model_type(self.hf_model_type)
        self.model_meta = get_model_meta(self.mcore_model_type)
        self.is_multimodal = self.model_meta.visual_cls is not None
        if self.is_multimodal and not self.language_model_only:
            self.test_mm_type = getattr(self.model_meta.visual_cls, 'test_mm_type', 'image')
        else:
            self.test_mm_type = 'text'
        if self.is_multimodal and self.hf_config is None:
            raise ValueError('Multimodal model must specify hf_config.')
        self.is_moe_model = self.num_moe_experts is not None
        self.bridge = self.model_meta.bridge_cls(self)

    # ------------------------------------------------------------------ helpers
    def _format_config(self):
        if self.window_size is not None:
            self.window_size = tuple_type(self.window_size)
        if self.window_attn_skip_freq is not None:
            self.window_attn_skip_freq = moe_freq_type(self.window_attn_skip_freq)
        if self.no_rope_freq is not None:
            self.no_rope_freq = no_rope_freq_type(self.no_rope_freq)
        if self.moe_layer_freq is not None:
            self.moe_layer_freq = moe_freq_type(self.moe_layer_freq)
        if self.linear_attention_freq is not None:
            self.linear_attention_freq = linear_attn_freq_type(self.linear_attention_freq)
            if isinstance(self.linear_attention_freq, int):
                n = self.linear_attention_freq
                self.linear_attention_freq = [0 if ((i + 1) % n == 0) else 1 for i in range(self.num_layers)]

    def _validate(self):
        tp = self.tensor_model_parallel_size
        if self.num_attention_heads is not None and self.num_attention_heads % tp != 0:
            raise ValueError(f'num_attention_heads ({self.num_attention_heads}) must be divisible by TP ({tp})')
        if self.num_moe_experts is not None and self.num_moe_experts % self.expert_model_parallel_size != 0:
            raise ValueError('num_moe_experts must be divisible by expert_model_parallel_size')
        if self.num_moe_experts and self.expert_model_parallel_size > 1 and self.tensor_model_parallel_size > 1 \
                and not self.sequence_parallel:
            # without sequence parallelism every tensor-parallel rank holds all tokens and would send each of them to
            # the experts once more: outputs would still be right, expert gradients would count every token tp times
            raise ValueError('expert parallelism together with tensor parallelism requires sequence_parallel=True')

    # pattern accessors (1-based semantics as in the reference's pattern language)
    def moe_layer_pattern(self) -> List[int]:
        """1 where layer i is an MoE layer."""
        n = self.num_layers
        if self.num_moe_experts is None:
            return [0] * n
        f = self.moe_layer_freq
        if isinstance(f, int):
            pat = [1 if (i % f == 0) else 0 for i in range(n)]
        else:
            pat = list(f)
            assert len(pat) == n, f'moe_layer_freq pattern length {len(pat)} != num_layers {n}'
        return pat

    def linear_attention_pattern(self) -> List[int]:
        """1 where layer i uses linear attention (gated DeltaNet), 0 for full attention."""
        if self.linear_attention_freq is None:
            return [0] * self.num_layers
        pat = list(self.linear_attention_freq)
        assert len(pat) == self.num_layers
        return pat

    def no_rope_pattern(self) -> List[int]:
        n = self.num_layers
        f = self.no_rope_freq
        if f is None:
            return [0] * n
        if isinstance(f, int):
            return [1 if ((i + 1) % f == 0) else 0 for i in range(n)]
        return list(f)

    def window_pattern(self) -> List[int]:
        """1 where layer i uses sliding-window attention."""
        n = self.num_layers
        if self.window_size is None:
            return [0] * n
        f = self.window_attn_skip_freq
        if f is None:
            return [1] * n
        if isinstance(f, int):
            return [0 if ((i + 1) % f == 0) else 1 for i in range(n)]
        return list(f)

    @property
    def head_dim(self) -> int:
        return self.kv_channels

    def __deepcopy__(self, memo):
        cls = self.__class__
        new_obj = cls.__new__(cls)
        memo[id(self)] = new_obj
        for k, v in self.__dict__.items():
            if k in ('bridge', 'model_meta', 'hf_config'):
                setattr(new_obj, k, v)
            else:
                setattr(new_obj, k, copy.deepcopy(v, memo))
        return new_obj
