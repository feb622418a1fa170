"""Configuration tree: nested dataclasses filled from ``key.sub=value`` command-line overrides.

The key names are the public contract shared with the reference
(skyrl/train/config/config.py:43-1762), so that a launch line written for it
(``trainer.algorithm.advantage_estimator=grpo generator.n_samples_per_prompt=8 ...``) works here.
The machinery is different: there is no OmegaConf; ``BaseConfig.from_dict`` walks the dataclass type
hints, coerces scalars parsed from the command line with YAML rules, rejects unknown keys with the
list of valid ones, and ``from_cli_overrides`` applies a dotlist on top of the defaults.
Extra knobs that only exist here (engine block size, fused-kernel toggles, packing and balancing)
live under ``trainer.b200``.
"""

from __future__ import annotations

import copy
import dataclasses
import os
import re
import typing
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Union

import yaml


class ConfigError(ValueError):
    pass


_FLOAT_RE = re.compile(r"^[+-]?\d+(\.\d*)?[eE][+-]?\d+$")


def _parse_scalar(text: str) -> Any:
    """Parse the right-hand side of ``key=value`` with YAML scalar/list/dict rules."""
    if text == "":
        return ""
    try:
        val = yaml.safe_load(text)
    except yaml.YAMLError:
        return text
    if isinstance(val, str) and _FLOAT_RE.match(text.strip()):
        return float(val)  # YAML 1.1 wants a dot in the mantissa ("1.0e-5"); people write "1e-5" (unquoted)
    return val


def _is_optional(tp) -> bool:
    return typing.get_origin(tp) is Union and type(None) in typing.get_args(tp)


def _coerce(value: Any, tp: Any, path: str) -> Any:
    origin = typing.get_origin(tp)
    if tp is Any or tp is typing.Any:
        return value
    if origin is Union:
        args = typing.get_args(tp)
        if value is None and type(None) in args:
            return None
        last_err = None
        for a in args:
            if a is type(None):
                continue
            try:
                return _coerce(value, a, path)
            except (ConfigError, TypeError, ValueError) as e:  # try the next member
                last_err = e
        raise ConfigError(f"{path}: cannot interpret {value!r} as {tp}: {last_err}")
    if origin is typing.Literal:
        if value not in typing.get_args(tp):
            raise ConfigError(f"{path}: {value!r} not in {typing.get_args(tp)}")
        return value
    if dataclasses.is_dataclass(tp):
        if isinstance(value, tp):
            return value
        if isinstance(value, dict):
            return tp.from_dict(value, _path=path)
        raise ConfigError(f"{path}: expected a mapping for {tp.__name__}, got {type(value).__name__}")
    if origin in (list, List):
        (inner,) = typing.get_args(tp) or (Any,)
        if isinstance(value, str):
            value = [v for v in value.split(",") if v != ""]
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"{path}: expected a list, got {value!r}")
        return [_coerce(v, inner, f"{path}[{i}]") for i, v in enumerate(value)]
    if origin in (dict, Dict) or tp is dict:
        if not isinstance(value, dict):
            raise ConfigError(f"{path}: expected a mapping, got {value!r}")
        return dict(value)
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str) and value.lower() in ("true", "false"):
            return value.lower() == "true"
        raise ConfigError(f"{path}: expected a bool, got {value!r}")
    if tp is int:
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected an int, got a bool")
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            return int(value)
        raise ConfigError(f"{path}: expected an int, got {value!r}")
    if tp is float:
        if isinstance(value, bool):
            raise ConfigError(f"{path}: expected a float, got a bool")
        if isinstance(value, (int, float)):
            return float(value)
        if isinstance(value, str):
            return float(value)
        raise ConfigError(f"{path}: expected a float, got {value!r}")
    if tp is str:
        if value is None:
            raise ConfigError(f"{path}: expected a string, got null")
        return str(value)
    return value


@dataclass
class BaseConfig:
    """Base of every config node: dict round-trip with strict keys."""

    @classmethod
    def from_dict(cls, data: Dict[str, Any], _path: str = ""):
        hints = typing.get_type_hints(cls)
        names = {f.name for f in dataclasses.fields(cls)}
        unknown = [k for k in data if k not in names]
        if unknown:
            where = _path or cls.__name__
            raise ConfigError(f"unknown key(s) {unknown} under '{where}'; valid keys: {sorted(names)}")
        kwargs = {}
        for f in dataclasses.fields(cls):
            if f.name in data:
                kwargs[f.name] = _coerce(data[f.name], hints[f.name], f"{_path}.{f.name}" if _path else f.name)
        return cls(**kwargs)

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def get(self, key: str, default=None):
        return getattr(self, key, default)

    def __getitem__(self, key: str):
        return getattr(self, key)

    def __contains__(self, key: str) -> bool:
        return hasattr(self, key)


# ----------------------------------------------------------------------------- data / model
@dataclass
class DataLoaderConfig(BaseConfig):
    num_workers: Optional[int] = None  # None: 8
    persistent_workers: bool = False

    def __post_init__(self):
        if self.num_workers is not None and self.num_workers < 0:
            raise ConfigError("data.dataloader.num_workers must be None or >= 0")
        if self.num_workers is None:
            self.num_workers = 8
        if self.persistent_workers and self.num_workers == 0:
            raise ConfigError("data.dataloader.persistent_workers requires num_workers > 0")


@dataclass
class DataConfig(BaseConfig):
    train_data: List[str] = field(default_factory=lambda: [os.path.expanduser("~/data/gsm8k/train.parquet")])
    val_data: List[str] = field(default_factory=lambda: [os.path.expanduser("~/data/gsm8k/validation.parquet")])
    dataloader: DataLoaderConfig = field(default_factory=DataLoaderConfig)


@dataclass
class SkyRLLoraConfig(BaseConfig):
    rank: int = 0
    alpha: int = 16
    dropout: float = 0.0
    lora_sync_path: str = "/tmp/skyrl_lora_sync"
    target_modules: str = "all-linear"
    exclude_modules: Optional[str] = None
    init_method: str = "kaiming"
    max_loras: int = 1
    max_cpu_loras: Optional[int] = None


@dataclass
class FakeInt4QatConfig(BaseConfig):
    enabled: bool = False
    group_size: int = 32
    symmetric: bool = True
    scale_divisor: float = 7.5
    q_min: float = -8.0
    bf16_base_path: Optional[str] = None


@dataclass
class ModelConfig(BaseConfig):
    path: Optional[str] = None
    lora: SkyRLLoraConfig = field(default_factory=SkyRLLoraConfig)
    fake_int4_qat: FakeInt4QatConfig = field(default_factory=FakeInt4QatConfig)


@dataclass
class OptimizerConfig(BaseConfig):
    lr: float = 1e-6
    adam_betas: List[float] = field(default_factory=lambda: [0.9, 0.999])
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    offload_after_step: bool = True
    num_warmup_steps: int = 0
    scheduler: str = "constant_with_warmup"


@dataclass
class MixedPrecisionConfig(BaseConfig):
    param_dtype: str = "bf16"
    reduce_dtype: str = "fp32"
    buffer_dtype: str = "fp32"


@dataclass
class FSDPConfig(BaseConfig):
    cpu_offload: bool = False
    reshard_after_forward: Union[bool, int] = True
    fsdp_size: int = -1
    mixed_precision: Optional[MixedPrecisionConfig] = None
    wrap_policy: dict = field(default_factory=dict)


@dataclass
class MegatronDDPConfig(BaseConfig):
    grad_reduce_in_fp32: bool = True
    overlap_grad_reduce: bool = False
    overlap_param_gather: bool = False
    average_in_collective: bool = True


@dataclass
class TorchProfilerConfig(BaseConfig):
    enable: bool = False
    ranks: List[int] = field(default_factory=lambda: [0])
    save_path: Optional[str] = None
    skip_first: int = 10
    wait: int = 0
    warmup: int = 1
    active: int = 1
    repeat: int = 1
    activities: List[str] = field(default_factory=lambda: ["cpu", "cuda"])
    record_shapes: bool = True
    profile_memory: bool = False
    with_stack: bool = True
    with_flops: bool = False
    with_modules: bool = False
    export_type: str = "chrome_trace"

    def validate(self) -> None:
        """Nothing is checked while the profiler is off.  When on: at least one rank, a local ``save_path``, activities
        out of cpu / cuda (any case), ``export_type`` chrome_trace or stacks (stacks needs ``with_stack``), a schedule
        with non-negative phases and at least one active step (reference: config.py ``TorchProfilerConfig.validate``)."""
        if not self.enable:
            return
        if not self.ranks:
            raise ConfigError("torch_profiler_config.ranks must be non-empty when the profiler is enabled")
        if not self.save_path:
            raise ConfigError("torch_profiler_config.save_path must be set when the profiler is enabled")
        if "://" in str(self.save_path):
            raise ConfigError(f"torch_profiler_config.save_path must be a local path, got '{self.save_path}'")
        if not self.activities:
            raise ConfigError("torch_profiler_config.activities must be non-empty")
        bad = [a for a in self.activities if str(a).lower() not in ("cpu", "cuda")]
        if bad:
            raise ConfigError(f"torch_profiler_config.activities: unknown {bad}; choose from ['cpu', 'cuda']")
        if self.export_type not in ("chrome_trace", "stacks"):
            raise ConfigError(f"torch_profiler_config.export_type must be 'chrome_trace' or 'stacks', got '{self.export_type}'")
        if self.export_type == "stacks" and not self.with_stack:
            raise ConfigError("torch_profiler_config.export_type='stacks' needs with_stack=true")
        for name in ("skip_first", "wait", "warmup", "repeat"):
            if getattr(self, name) < 0:
                raise ConfigError(f"torch_profiler_config.{name} must be >= 0")
        if self.active < 1:
            raise ConfigError("torch_profiler_config.active must be >= 1")


@dataclass
class MegatronHFExportConfig(BaseConfig):
    distributed_save: bool = False
    save_every_n_ranks: int = 1


@dataclass
class MegatronLoraConfig(BaseConfig):
    lora_type: str = "lora"
    merge_lora: bool = True


@dataclass
class MegatronConfig(BaseConfig):
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    moe_token_dispatcher_type: str = "alltoall"
    moe_router_load_balancing_type: str = "none"
    moe_aux_loss_coeff: float = 0.0
    moe_grouped_gemm: bool = True
    moe_router_score_function: Optional[str] = None
    moe_router_enable_expert_bias: Optional[bool] = None
    moe_enable_routing_replay: bool = False
    moe_per_layer_logging: bool = False
    moe_router_dtype: str = "fp32"
    ddp_config: MegatronDDPConfig = field(default_factory=MegatronDDPConfig)
    hf_export_config: MegatronHFExportConfig = field(default_factory=MegatronHFExportConfig)
    lora_config: MegatronLoraConfig = field(default_factory=MegatronLoraConfig)
    optimizer_config_kwargs: Dict[str, Any] = field(default_factory=dict)
    transformer_config_kwargs: Dict[str, Any] = field(default_factory=dict)
    empty_cuda_cache: Optional[bool] = True
    model_config_kwargs: dict = field(default_factory=dict)
    dist_ckpt_optim_fully_reshardable: bool = False
    freeze_moe_router: bool = False
    mtp_num_layers: Optional[int] = None
    mtp_loss_weight: float = 0.1
    mtp_loss_chunk_size: Optional[int] = 1024
    mtp_loss_topk: Optional[int] = None
    async_dist_ckpt_save: bool = False
    async_dist_ckpt_strategy: str = "mcore"
    async_save_prestage_to_cpu: bool = False


@dataclass
class PlacementConfig(BaseConfig):
    colocate_all: bool = True
    colocate_policy_ref: bool = True
    policy_num_nodes: int = 1
    policy_num_gpus_per_node: int = 1
    critic_num_nodes: int = 1
    critic_num_gpus_per_node: int = 1
    ref_num_nodes: int = 1
    ref_num_gpus_per_node: int = 1


@dataclass
class PolicyConfig(BaseConfig):
    model: ModelConfig = field(default_factory=lambda: ModelConfig(path="Qwen/Qwen2.5-1.5B-Instruct"))
    optimizer_config: OptimizerConfig = field(default_factory=OptimizerConfig)
    fsdp_config: FSDPConfig = field(default_factory=FSDPConfig)
    sequence_parallel_size: int = 1
    use_torch_compile: bool = False
    record_memory: bool = False
    torch_profiler_config: TorchProfilerConfig = field(default_factory=TorchProfilerConfig)
    megatron_config: MegatronConfig = field(default_factory=MegatronConfig)
    model_config_kwargs: dict = field(default_factory=dict)
    language_model_only: bool = False
    inference_only_init: bool = False


@dataclass
class CriticConfig(BaseConfig):
    model: ModelConfig = field(default_factory=ModelConfig)
    optimizer_config: OptimizerConfig = field(default_factory=lambda: OptimizerConfig(lr=5e-6))
    fsdp_config: FSDPConfig = field(default_factory=FSDPConfig)
    sequence_parallel_size: int = 1
    model_config_kwargs: dict = field(default_factory=dict)
    megatron_config: MegatronConfig = field(default_factory=MegatronConfig)


@dataclass
class RefConfig(BaseConfig):
    model: ModelConfig = field(default_factory=ModelConfig)
    sequence_parallel_size: int = 1
    fsdp_config: FSDPConfig = field(default_factory=FSDPConfig)
    megatron_config: MegatronConfig = field(default_factory=MegatronConfig)
    model_config_kwargs: dict = field(default_factory=dict)
    language_model_only: bool = False


# ----------------------------------------------------------------------------- algorithm
@dataclass
class KLCtrlConfig(BaseConfig):
    type: str = "fixed"
    kl_target: float = 0.1
    horizon: int = 10000


@dataclass
class SAPOConfig(BaseConfig):
    tau_pos: float = 1.0
    tau_neg: float = 1.05


@dataclass
class DynamicSamplingConfig(BaseConfig):
    type: Optional[str] = None
    max_sample_batches: int = 30
    min_replace_ratio: float = 0.3


@dataclass
class ClipCovConfig(BaseConfig):
    clip_ratio: float = 0.0002
    clip_cov_lb: float = 1.0
    clip_cov_ub: float = 5.0


@dataclass
class KLCovConfig(BaseConfig):
    kl_cov_frac: float = 0.2
    ppo_kl_coef: float = 1.0


@dataclass
class CISPOConfig(BaseConfig):
    cispo_eps_clip_low: float = 1.0
    cispo_eps_clip_high: float = 4.0
    cispo_anchor: str = "old"


@dataclass
class DPPOConfig(BaseConfig):
    dppo_type: str = "binary_tv"
    delta_low: float = 0.2
    delta_high: float = 0.2


@dataclass
class OffPolicyCorrectionConfig(BaseConfig):
    tis_ratio_type: Optional[str] = None
    token_tis_ratio_clip_high: float = 2.0
    sequence_tis_ratio_clip_high: float = 5.0
    sequence_mask_metric: Optional[str] = None
    geo_mask_high: float = 1.01
    geo_mask_low: float = 0.99
    product_mask_high: float = 2.0
    product_mask_low: float = 0.5
    outlier_token_is_threshold_low: Optional[float] = None
    outlier_token_is_threshold_high: Optional[float] = None
    token_mask_is_threshold_low: Optional[float] = None
    token_mask_is_threshold_high: Optional[float] = None


@dataclass
class AlgorithmConfig(BaseConfig):
    advantage_estimator: str = "grpo"
    kl_ctrl: KLCtrlConfig = field(default_factory=KLCtrlConfig)
    kl_estimator_type: str = "k3"
    use_kl_in_reward: bool = False
    use_kl_loss: bool = True
    kl_loss_coef: float = 0.001
    use_entropy_loss: bool = False
    entropy_loss_coef: float = 0.01
    temperature: Optional[float] = None
    advantage_batch_normalize: bool = False
    value_head_prefix: str = "value_head"
    policy_loss_type: str = "regular"
    loss_reduction: str = "token_mean"
    grpo_norm_by_std: bool = True
    zero_variance_filter: bool = False
    zero_variance_filter_tol: float = 1e-6
    lambd: float = 1.0
    gamma: float = 1.0
    eps_clip_low: float = 0.2
    eps_clip_high: float = 0.2
    clip_ratio_c: float = 3.0
    tis_imp_ratio_cap: float = -1.0
    use_tis: bool = False
    off_policy_correction: OffPolicyCorrectionConfig = field(default_factory=OffPolicyCorrectionConfig)
    sapo: SAPOConfig = field(default_factory=SAPOConfig)
    value_clip: Optional[float] = 0.2
    dynamic_sampling: DynamicSamplingConfig = field(default_factory=DynamicSamplingConfig)
    clip_cov: ClipCovConfig = field(default_factory=ClipCovConfig)
    kl_cov: KLCovConfig = field(default_factory=KLCovConfig)
    cispo: CISPOConfig = field(default_factory=CISPOConfig)
    dppo: DPPOConfig = field(default_factory=DPPOConfig)
    max_seq_len: Optional[int] = None


@dataclass
class FullyAsyncConfig(BaseConfig):
    enabled: bool = False
    max_staleness_steps: int = 4
    num_parallel_generation_workers: int = 768
    sample_full_batch: bool = False
    clear_kv_cache_on_weight_sync: bool = False
    simulate_training: bool = False
    simulate_training_step_seconds: float = 30.0
    simulate_weight_sync_seconds: float = 0.0


# ----------------------------------------------------------------------------- generator / engine
@dataclass
class SamplingParams(BaseConfig):
    max_generate_length: int = 1024
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    min_p: float = 0.0
    top_k: int = -1
    logprobs: Optional[int] = 1
    stop: Optional[List[str]] = None
    additional_kwargs: Optional[Dict[str, Any]] = None


@dataclass
class ChatTemplateConfig(BaseConfig):
    source: str = "name"
    name_or_path: Optional[str] = None


@dataclass
class DeltaWeightSyncConfig(BaseConfig):
    sync_dir: str = ""
    local_checkpoint_dir: Optional[str] = None
    publish_staging_dir: Optional[str] = None
    max_file_size_in_gb: float = 1.0
    cloud_download_workers: int = 4
    publish_num_workers: Optional[int] = None
    checkpoint_load_format: str = "multi_thread_safetensors"
    multi_thread_safetensors_max_workers: int = 8


@dataclass
class InferenceEngineConfig(BaseConfig):
    model_dtype: str = "bfloat16"
    run_engines_locally: bool = True
    num_engines: int = 1
    backend: str = "b200"
    weight_sync_backend: str = "nccl"
    weight_transfer_threshold_cuda_ipc_GB: float = 1.0
    delta_weight_sync: Optional[DeltaWeightSyncConfig] = None
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    expert_parallel_size: int = 1
    data_parallel_size: int = 1
    vllm_v1_disable_multiproc: bool = True
    enable_prefix_caching: bool = True
    enable_chunked_prefill: bool = True
    enable_return_routed_experts: bool = False
    max_num_batched_tokens: int = 8192
    enforce_eager: bool = False
    fully_sharded_loras: bool = False
    enable_ray_prometheus_stats: bool = True
    gpu_memory_utilization: float = 0.8
    offload_kv_for_weight_sync: bool = False
    use_expandable_segments: bool = False
    max_num_seqs: int = 1024
    served_model_name: Optional[str] = None
    distributed_executor_backend: str = "mp"
    language_model_only: bool = False
    engine_init_kwargs: Dict[str, Any] = field(default_factory=dict)
    speculative_config: Optional[Dict[str, Any]] = None
    external_proxy_url: Optional[str] = None
    external_server_urls: Optional[List[str]] = None
    enable_pd: bool = False
    num_prefill: int = 0
    router_init_kwargs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class GeneratorConfig(BaseConfig):
    inference_engine: InferenceEngineConfig = field(default_factory=InferenceEngineConfig)
    n_samples_per_prompt: int = 5
    batched: bool = False
    max_turns: int = 1
    max_input_length: Optional[int] = None
    chat_template: ChatTemplateConfig = field(default_factory=ChatTemplateConfig)
    chat_template_kwargs: Dict[str, Any] = field(default_factory=dict)
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    use_conversation_multi_turn: bool = True
    append_eos_token_after_stop_str_in_multi_turn: bool = True
    eval_sampling_params: Optional[SamplingParams] = None
    eval_n_samples_per_prompt: int = 1
    zero_reward_on_non_stop: bool = False
    use_cache_salt: bool = True
    apply_overlong_filtering: bool = False
    step_wise_trajectories: bool = False
    vision_language_generator: bool = False
    merge_stepwise_output: bool = False


@dataclass
class Text2SQLEnvConfig(BaseConfig):
    db_path: str = ""


@dataclass
class GSM8kLLMJudgeEnvConfig(BaseConfig):
    model: str = "gpt-4o-mini"
    base_url: Optional[str] = None


@dataclass
class SearchEnvConfig(BaseConfig):
    log_requests: bool = False
    search_url: str = "http://127.0.0.1:8000/retrieve"
    topk: int = 3
    timeout: int = 30


@dataclass
class SkyRLGymConfig(BaseConfig):
    max_env_workers: int = 32
    text2sql: Text2SQLEnvConfig = field(default_factory=Text2SQLEnvConfig)
    llm_as_a_judge: GSM8kLLMJudgeEnvConfig = field(default_factory=GSM8kLLMJudgeEnvConfig)
    search: SearchEnvConfig = field(default_factory=SearchEnvConfig)


@dataclass
class EnvironmentConfig(BaseConfig):
    env_class: str = "gsm8k"
    skyrl_gym: SkyRLGymConfig = field(default_factory=SkyRLGymConfig)


@dataclass
class MTPConfig(BaseConfig):
    enabled: bool = False
    num_speculative_tokens: int = 1
    loss_weight: float = 0.1


@dataclass
class B200Config(BaseConfig):
    """Knobs of this implementation that the reference has no equivalent for."""

    kv_block_size: int = 32
    fused_optimizer: bool = True  # reduce-scatter + AdamW + parameter push in one peer-memory kernel
    cuda_graph_decode: bool = True
    # with trainer.mtp.enabled: the colocated engine drafts one token per step with the draft head being trained
    # (decode steps then run eagerly, two rows per sequence); false keeps plain decoding and only trains the head
    speculative_decode: bool = True
    # batch sizes the engine captures decode graphs for (a step runs at the smallest one that holds its live slots);
    # empty = the engine's own ladder
    decode_graph_batch_sizes: List[int] = field(default_factory=list)
    # With exactly one optimizer step per RL step the "old policy" is the policy being trained, so its
    # log-probabilities are the (detached) ones of the training forward pass: no separate forward is run.
    reuse_train_forward_for_old_logprobs: bool = True
    # packed micro-batches are padded (one dummy sequence) to a multiple of this many tokens so that activation
    # tensors repeat in size from step to step; 0 disables
    pack_pad_multiple: int = 512
    # "full": token-budget micro-batches are filled to the budget (first-fit decreasing) and padded to exactly the
    # budget, so activation sizes repeat; "balanced": equal-load bins (the reference's packer)
    microbatch_packing: str = "full"
    # tensor-parallel training: shard the LM head over the vocabulary (fused log-prob kernel per shard, softmax records
    # merged across ranks through peer memory) instead of over the tokens; needs untied embeddings
    vocab_parallel_lm_head: bool = False
    # fused peer optimizer: start each layer's gradient reduce-scatter behind the last micro-batch's backward pass
    overlap_grad_reduce: bool = True
    # pure data parallelism: re-deal the rows of every policy mini-batch among the ranks so that all ranks train on
    # about the same number of tokens (the summed gradient does not change; train/balance.py)
    balance_tokens_across_ranks: bool = True


@dataclass
class TrainerConfig(BaseConfig):
    placement: PlacementConfig = field(default_factory=PlacementConfig)
    use_expandable_segments: bool = True
    sequence_parallel_backend: str = "ulysses"
    strategy: str = "fsdp"
    policy: PolicyConfig = field(default_factory=PolicyConfig)
    ref: RefConfig = field(default_factory=RefConfig)
    critic: CriticConfig = field(default_factory=CriticConfig)
    algorithm: AlgorithmConfig = field(default_factory=AlgorithmConfig)
    mtp: MTPConfig = field(default_factory=MTPConfig)
    fully_async: FullyAsyncConfig = field(default_factory=FullyAsyncConfig)
    b200: B200Config = field(default_factory=B200Config)
    gradient_checkpointing: bool = True
    gradient_checkpointing_use_reentrant: bool = False
    seed: int = 42
    resume_mode: Optional[str] = "latest"
    resume_path: Optional[str] = None
    log_path: str = "/tmp/skyrl-logs"
    ckpt_path: str = field(default_factory=lambda: os.path.expanduser("~/ckpts/"))
    max_ckpts_to_keep: int = -1
    ckpt_interval: int = 10
    hf_save_interval: int = -1
    export_path: str = field(default_factory=lambda: os.path.expanduser("~/exports/"))
    bf16: bool = True
    epochs: int = 1
    max_training_steps: Optional[int] = None
    update_epochs_per_batch: int = 1
    train_batch_size: int = 1024
    policy_mini_batch_size: int = 256
    critic_mini_batch_size: int = 256
    micro_train_batch_size_per_gpu: int = 1
    micro_forward_batch_size_per_gpu: int = 1
    max_tokens_per_microbatch: int = -1
    recompute_old_logprobs_per_minibatch: bool = True
    update_ref_every_epoch: bool = False
    remove_microbatch_padding: bool = True
    eval_batch_size: int = 1024
    eval_before_train: bool = True
    eval_interval: int = 5
    max_prompt_length: int = 512
    flash_attn: bool = True
    disable_fast_tokenizer: bool = False
    project_name: str = "skyrl"
    run_name: str = "test_run"
    logger: str = "console"
    enable_ray_gpu_monitor: bool = True
    tags: Optional[List[str]] = None
    dump_data_batch: bool = False
    dump_eval_results: bool = True
    print_example_interval: int = 1
    num_logger_eval_samples: int = -1
    num_logger_train_samples: int = -1
    log_example_interval: int = -1
    logprobs_chunk_size: Optional[int] = 1024
    vocab_entropy_chunk_size: Optional[int] = 0
    vocab_entropy_chunk_memory_mb: int = 512
    fused_lm_head_logprob: bool = True
    fused_lm_head_logprob_backend: str = "tcgen05"
    override_entrypoint: Optional[str] = None


@dataclass
class SkyRLTrainConfig(BaseConfig):
    data: DataConfig = field(default_factory=DataConfig)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    generator: GeneratorConfig = field(default_factory=GeneratorConfig)
    environment: EnvironmentConfig = field(default_factory=EnvironmentConfig)

    def __post_init__(self):
        self._derive()

    def _derive(self) -> None:
        g, t = self.generator, self.trainer
        if g.max_input_length is None:
            g.max_input_length = t.max_prompt_length + g.sampling_params.max_generate_length * max(1, g.max_turns - 1)
        if t.algorithm.temperature is None:
            t.algorithm.temperature = g.sampling_params.temperature
        if t.algorithm.max_seq_len is None:
            t.algorithm.max_seq_len = g.max_input_length + g.sampling_params.max_generate_length
        if g.eval_sampling_params is None:
            g.eval_sampling_params = copy.deepcopy(g.sampling_params)
        if t.log_example_interval > 0:  # old name of print_example_interval
            t.print_example_interval = t.log_example_interval
        if t.ref.model.path is None:
            t.ref.model.path = t.policy.model.path

    # ------------------------------------------------------------------ CLI
    _RENAMED = {
        "trainer.use_sample_packing": "trainer.remove_microbatch_padding",
        "generator.backend": "generator.inference_engine.backend",
        "generator.num_inference_engines": "generator.inference_engine.num_engines",
        "generator.inference_engine_tensor_parallel_size": "generator.inference_engine.tensor_parallel_size",
        "generator.gpu_memory_utilization": "generator.inference_engine.gpu_memory_utilization",
        "generator.weight_sync_backend": "generator.inference_engine.weight_sync_backend",
        "generator.run_engines_locally": "generator.inference_engine.run_engines_locally",
        "generator.enable_prefix_caching": "generator.inference_engine.enable_prefix_caching",
        "generator.max_num_seqs": "generator.inference_engine.max_num_seqs",
        "generator.max_num_batched_tokens": "generator.inference_engine.max_num_batched_tokens",
        "generator.enforce_eager": "generator.inference_engine.enforce_eager",
    }

    @classmethod
    def from_cli_overrides(cls, args: Union[List[str], Dict[str, Any]]) -> "SkyRLTrainConfig":
        """Build a config from ``a.b.c=value`` strings, or from a ``{"a.b.c": value}`` mapping whose values keep their
        Python types (``None`` stays ``None``, ``"1e-5"`` stays a string) instead of going through the text parser
        (reference: config.py:1765-1891)."""
        tree: Dict[str, Any] = {}
        typed = isinstance(args, dict)
        for raw in (args.items() if typed else args):
            if typed:
                key, val = raw
                raw = f"{key}=..."
            else:
                if "=" not in raw:
                    if raw.startswith("+"):
                        raise ConfigError(f"'+' overrides are not supported: {raw!r}; every key must already exist")
                    raise ConfigError(f"override {raw!r} is not of the form key=value")
                key, val = raw.split("=", 1)
            if str(key).startswith("+"):
                raise ConfigError(f"'+' overrides are not supported: {key!r}; every key must already exist")
            key = str(key).strip().lstrip("-")
            key = cls._RENAMED.get(key, key)
            parts = key.split(".")
            node = tree
            for p in parts[:-1]:
                nxt = node.setdefault(p, {})
                if not isinstance(nxt, dict):
                    raise ConfigError(f"override {raw!r} conflicts with an earlier scalar value for '{p}'")
                node = nxt
            parsed = val if typed else _parse_scalar(val)
            if parts[-1] == "strategy" and parsed == "fsdp2":
                parsed = "fsdp"
            node[parts[-1]] = parsed
        return cls.from_nested(tree)

    @classmethod
    def from_nested(cls, tree: Dict[str, Any]) -> "SkyRLTrainConfig":
        base = cls().to_dict()
        # derived values must be recomputed from the overridden inputs, so drop the defaults' derivations
        base["generator"]["max_input_length"] = None
        base["generator"]["eval_sampling_params"] = None
        base["trainer"]["algorithm"]["temperature"] = None
        base["trainer"]["algorithm"]["max_seq_len"] = None
        base["trainer"]["ref"]["model"]["path"] = None
        merged = _deep_merge(base, tree, path="")
        return cls.from_dict(merged)


def overrides_dict_to_dotlist(overrides: Dict[str, Any]) -> List[str]:
    """``{"a.b": value}`` -> ``["a.b=<text>"]`` such that parsing the text gives the value back: ``None`` -> ``null``,
    booleans lower-case, containers and strings as JSON (so ``"1e-5"`` or ``"null"`` stay strings); anything JSON
    cannot express falls back to ``str`` (reference: config.py, same name)."""
    import json

    out = []
    for k, v in overrides.items():
        if v is None:
            text = "null"
        elif isinstance(v, bool):
            text = "true" if v else "false"
        elif isinstance(v, (int, float)):
            text = repr(v)
        else:
            try:
                text = json.dumps(v)
            except (TypeError, ValueError):
                text = str(v)
        out.append(f"{k}={text}")
    return out


def _deep_merge(base: Dict[str, Any], over: Dict[str, Any], path: str) -> Dict[str, Any]:
    out = dict(base)
    for k, v in over.items():
        here = f"{path}.{k}" if path else k
        if k not in base:
            # free-form dict fields accept new keys; everything else is validated by from_dict
            out[k] = v
        elif isinstance(base[k], dict) and isinstance(v, dict):
            out[k] = _deep_merge(base[k], v, here)
        else:
            out[k] = v
    return out


def make_config(**section_classes) -> type:
    """Create a ``SkyRLTrainConfig`` subclass whose sections use extended dataclasses.

    ``make_config(trainer=MyTrainerConfig)`` mirrors the reference helper (config.py:1894-1951) for
    users who add their own keys.
    """
    hints = typing.get_type_hints(SkyRLTrainConfig)
    fields_ = []
    for f in dataclasses.fields(SkyRLTrainConfig):
        tp = section_classes.get(f.name, hints[f.name])
        fields_.append((f.name, tp, field(default_factory=tp)))
    unknown = set(section_classes) - {f.name for f in dataclasses.fields(SkyRLTrainConfig)}
    if unknown:
        raise ConfigError(f"make_config: unknown section(s) {sorted(unknown)}")
    return dataclasses.make_dataclass("CustomSkyRLTrainConfig", fields_, bases=(SkyRLTrainConfig,))


def get_config_as_yaml_str(cfg: BaseConfig) -> str:
    return yaml.safe_dump(cfg.to_dict(), sort_keys=False)
