"""SFT configuration (reference: skyrl/train/config/sft_config.py:33-697).  Same key names where the concept
carries over; keys that configure Ray placement or the Megatron backend are accepted and mapped onto the single
process-per-GPU runtime (``placement.num_gpus_per_node`` must match the launched world size)."""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .config import (BaseConfig, ConfigError, FSDPConfig, MegatronConfig, ModelConfig, OptimizerConfig,
                     TorchProfilerConfig, _parse_scalar)

TRAIN_ON_LAST = "last_assistant_message"
TRAIN_ON_ALL = "all_assistant_messages"


@dataclass
class SFTPlacementConfig(BaseConfig):
    num_nodes: int = 1
    num_gpus_per_node: int = 1


@dataclass
class SFTConfig(BaseConfig):
    model: ModelConfig = field(default_factory=lambda: ModelConfig(path="tiny-qwen2-d128"))
    optimizer_config: OptimizerConfig = field(default_factory=OptimizerConfig)
    placement: SFTPlacementConfig = field(default_factory=SFTPlacementConfig)
    megatron_config: MegatronConfig = field(default_factory=MegatronConfig)
    fsdp_config: FSDPConfig = field(default_factory=FSDPConfig)
    sequence_parallel_size: int = 1
    model_config_kwargs: Dict[str, Any] = field(default_factory=dict)
    use_torch_compile: bool = False  # accepted for compatibility; the hot path is hand-written kernels
    record_memory: bool = False
    torch_profiler_config: TorchProfilerConfig = field(default_factory=TorchProfilerConfig)
    strategy: str = "fsdp"
    # --- data
    dataset_name: Optional[str] = None
    dataset_split: Optional[str] = None
    train_datasets: Optional[List[str]] = None
    train_dataset_splits: Optional[List[str]] = None
    train_dataset_weights: Optional[List[float]] = None
    pretokenized_dataset_paths: Optional[List[str]] = None
    messages_key: str = "messages"
    tools_key: str = "tools"
    system_key: str = "system"
    eval_dataset_name: Optional[str] = None
    eval_dataset_split: Optional[str] = None
    eval_datasets: Optional[List[str]] = None
    eval_dataset_splits: Optional[List[str]] = None
    eval_dataset_names: Optional[List[str]] = None
    eval_pretokenized_dataset_paths: Optional[List[str]] = None
    eval_interval: int = 0
    eval_before_train: bool = False
    max_length: Optional[int] = None
    # --- schedule
    num_steps: Optional[int] = None
    num_epochs: Optional[int] = 1
    max_training_steps: Optional[int] = None
    batch_size: int = 4
    micro_train_batch_size_per_gpu: int = 2
    # --- logging / checkpoints
    logger: str = "console"
    project_name: str = "skyrl_sft"
    run_name: str = "skyrl_sft_run"
    tags: Optional[List[str]] = None
    log_path: str = "/tmp/skyrl-logs"
    ckpt_path: str = ""
    ckpt_interval: int = 0
    enable_ray_gpu_monitor: bool = True
    max_ckpts_to_keep: int = -1
    resume_from: str = ""
    hf_save_interval: int = 0
    export_path: str = ""
    seed: int = 42
    # --- tokenization / loading
    num_workers: int = 8
    async_batch_collation: bool = True
    dataloader_num_workers: int = 0
    dataloader_persistent_workers: bool = False
    sampler: str = "random"  # "random" | "sequential" | "length_grouped"
    sampler_class_path: Optional[str] = None
    sampler_kwargs: Dict[str, Any] = field(default_factory=dict)
    cache_dir: str = field(default_factory=lambda: os.path.join(os.path.expanduser("~"), ".cache", "skyrl_b200", "sft"))
    force_recache: bool = False
    disable_cache: bool = False
    train_on_what: str = TRAIN_ON_LAST
    # --- batching
    remove_microbatch_padding: bool = True
    use_sequence_packing: bool = False
    max_tokens_per_microbatch: Optional[int] = None
    bf16: bool = True
    gradient_checkpointing: bool = False
    # --- dummy run
    dummy_run_full_ctx: bool = False
    dummy_run_max_steps: int = 5

    def __post_init__(self):
        if self.train_on_what not in (TRAIN_ON_LAST, TRAIN_ON_ALL):
            raise ConfigError(f"train_on_what must be '{TRAIN_ON_LAST}' or '{TRAIN_ON_ALL}', got {self.train_on_what!r}")
        if self.strategy == "fsdp2":
            self.strategy = "fsdp"
        if self.strategy not in ("fsdp", "megatron"):
            raise ConfigError(f"strategy must be 'fsdp' or 'megatron', got {self.strategy!r}")
        if self.dataset_name and self.train_datasets:
            raise ConfigError("give either dataset_name or train_datasets, not both")
        if self.train_dataset_weights is not None:
            n = len(self.train_datasets or [])
            if len(self.train_dataset_weights) != n:
                raise ConfigError(f"train_dataset_weights has {len(self.train_dataset_weights)} entries for {n} datasets")
            if any(w <= 0 for w in self.train_dataset_weights):
                raise ConfigError("train_dataset_weights must be positive")
        if self.use_sequence_packing and not self.max_tokens_per_microbatch and not self.max_length:
            raise ConfigError("use_sequence_packing needs max_tokens_per_microbatch (or max_length) as the bin capacity")
        if self.batch_size <= 0 or self.micro_train_batch_size_per_gpu <= 0:
            raise ConfigError("batch_size and micro_train_batch_size_per_gpu must be positive")

    def train_sources(self) -> List[str]:
        if self.train_datasets:
            return list(self.train_datasets)
        return [self.dataset_name] if self.dataset_name else []

    def eval_sources(self) -> List[str]:
        if self.eval_datasets:
            return list(self.eval_datasets)
        return [self.eval_dataset_name] if self.eval_dataset_name else []

    @classmethod
    def from_cli_overrides(cls, args: List[str]) -> "SFTConfig":
        tree: Dict[str, Any] = {}
        for raw in args:
            if raw.startswith("+") or "=" not in raw:
                raise ConfigError(f"override {raw!r} is not of the form key=value ('+' keys are not supported)")
            key, val = raw.split("=", 1)
            node = tree
            parts = key.strip().lstrip("-").split(".")
            for p in parts[:-1]:
                node = node.setdefault(p, {})
            node[parts[-1]] = _parse_scalar(val)
        return cls.from_dict(tree)
