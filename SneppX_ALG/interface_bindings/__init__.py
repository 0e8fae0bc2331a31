"""Flat re-export with the reference's public names (interface_bindings/__init__.py of the reference lists them per
module).  A name resolves lazily on first access so that importing the shim stays cheap."""
import importlib

_WHERE = {
    # nn
    **{n: "nn" for n in ("Module", "Linear", "Embedding", "Dropout", "LayerNorm", "RMSNorm", "GELU", "SiLU", "ReLU",
                         "Sigmoid", "Tanh", "Sequential", "MultiheadAttention", "TransformerBlock", "Transformer")},
    **{n: "nn.attention" for n in ("Attention", "DifferentialAttention", "FlexAttention", "SlidingWindowAttention",
                                   "SparseAttention", "ALiBiAttention", "CrossAttention", "MultiHeadLatentAttention",
                                   "MixtureOfDepths")},
    "Mamba2": "nn.ssm",
    # optim / schedulers
    **{n: "optim.zoo" for n in ("SGD", "AdamW", "Lion", "LAMB", "LARS", "AdaFactor", "SM3", "SOAP", "DistributedAdam", "Demeter", "CaProp", "OrthoAdam",
                                "get_optimizer")},
    **{n: "training.schedulers" for n in ("CosineAnnealingLR", "get_scheduler")},
    # training
    **{n: "training.config" for n in ("TrainConfig",)},
    **{n: "training.trainer" for n in ("Trainer",)},
    **{n: "training.amp" for n in ("autocast", "GradScaler")},
    **{n: "training.lora" for n in ("LoRALinear", "apply_lora", "DPOTrainer", "GRPOTrainer")},
    **{n: "training.data" for n in ("DataLoader", "MemoryMappedTextDataset", "StreamingTokenDataset", "DistributedSampler")},
    # distributed
    **{n: "parallel.distributed" for n in ("init_process_group", "destroy_process_group", "get_world_size", "get_rank",
                                           "barrier", "all_reduce", "broadcast", "DistributedContext",
                                           "DistributedDataParallel", "launch", "ProcessGroup")},
    **{n: "parallel.fsdp" for n in ("FullyShardedDataParallel", "FSDPConfig", "ShardingStrategy", "MixedPrecision",
                                    "shard_model", "fsdp_save_checkpoint", "fsdp_load_checkpoint")},
    # checkpoint / fault tolerance
    **{n: "checkpoint.sneppx_format" for n in ("CheckpointWriter", "CheckpointReader", "validate_checkpoint")},
    **{n: "checkpoint.manager" for n in ("CheckpointManager", "CheckpointCoordinator")},
    **{n: "parallel.host_runtime" for n in ("HeartbeatMonitor", "ElasticTrainer", "FaultToleranceManager")},
    # algorithms
    **{n: "algorithms" for n in ("Model", "ModelConfig", "HSSConfig", "HSSModel", "HSSDiscretize", "HSSScan", "HSSStep",
                                 "SERConfig", "SERModel", "SERLayer", "SERRoute", "SERLoss", "ARCConfig", "ARCModel",
                                 "NPEConfig", "NPEModel", "FMConfig", "FMModel", "FMSyncNCCL")},
    # models / zoo / hub
    **{n: "models" for n in ("LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM", "create_model", "LlamaConfig",
                             "MistralConfig", "Qwen2Config", "DeepSeekV2Config", "get_model_config", "extend_context")},
    "DeepSeekV2ForCausalLM": "models.deepseek",
    **{n: "models.families" for n in ("BertModel", "BertForMaskedLM", "GPTModel", "GPT2LMHeadModel",
                                      "T5ForConditionalGeneration", "VisionTransformer")},
    **{n: "hub.model_hub" for n in ("from_pretrained", "ModelHub", "convert_hf_to_sneppx", "Hub")},
    # quantisation
    **{n: "quant" for n in ("QuantMode", "quantize_int8", "awq_quantize", "gptq_quantize", "QuantizedLinear",
                            "mx_quantize", "nvfp4_quantize")},
    # serving
    **{n: "serving.kv_cache" for n in ("KVBlockPool", "PagedKVCache", "PrefixCache")},
    **{n: "serving.generation" for n in ("generate", "greedy_search", "beam_search", "batch_generate")},
    **{n: "serving.serving_engine" for n in ("ServingEngine",)},
    **{n: "serving.server" for n in ("create_app",)},
    **{n: "training.keras_api" for n in ("UltraTrainer",)},
    **{n: "serving.middleware" for n in ("SecurityMiddleware",)},
    **{n: "serving.watermark" for n in ("Watermark",)},
    **{n: "serving.client" for n in ("ServingClient",)},
    **{n: "utils.vizmon" for n in ("VizMon",)},
    **{n: "utils.registry" for n in ("ModelRegistry", "PromptRegistry")},
    **{n: "security.services" for n in ("KeyVault", "AuditLogger", "DDoSMitigator", "Firewall", "IntegrityMonitor",
                                        "ApiKeyStore", "UsageTracker")},
    **{n: "security.ai_filter" for n in ("PromptFilter", "OutputVerifier")},
    **{n: "hub.hf" for n in ("from_huggingface", "to_huggingface", "pipeline", "load_hf_dataset", "load_hf_model",
                             "save_hf_model")},
    **{n: "jit" for n in ("trace", "grad", "vmap", "jacobian", "hessian")},
    **{n: "tensor" for n in ("Tensor", "Function", "Context", "no_grad")},
    # names that live in a module of the same meaning under another path
    **{n: 'algorithms.fm' for n in ('FMController',)},
    **{n: 'algorithms.npe' for n in ('NPEProgram', 'NPEVM')},
    **{n: 'cli' for n in ('serve_main',)},
    **{n: 'device' for n in ('device_count', 'set_device', 'synchronize')},
    **{n: 'hub' for n in ('HF_WEIGHT_MAP',)},
    **{n: 'jit' for n in ('value_and_grad',)},
    **{n: 'models.config' for n in ('list_models',)},
    **{n: 'models.families' for n in ('BertConfig', 'GPTConfig', 'T5Config')},
    **{n: 'models.llama' for n in ('LlamaAttention', 'LlamaMLP')},
    **{n: 'onnx.toolkit' for n in ('infer_shapes',)},
    **{n: 'ops.functional' for n in ('layernorm', 'rmsnorm')},
    **{n: 'optim.fused' for n in ('clip_grad_norm_',)},
    **{n: 'optim.zoo' for n in ('Optimizer', 'RAdam', 'ScheduleFreeAdamW')},
    **{n: 'parallel.distributed' for n in ('DistributedWrapper',)},
    **{n: 'security.crypto' for n in ('sha256', 'sha3_256', 'sha3_512', 'sha512')},
    **{n: 'security.services' for n in ('TokenBucket',)},
    **{n: 'serving.generation' for n in ('sample_generation', 'top_k_top_p_filtering')},
    **{n: 'serving.serving_engine' for n in ('MetricsCollector', 'ModelVersion')},
    **{n: 'tensor' for n in ('avg_pool2d', 'conv1d', 'conv2d', 'max_pool2d', 'softmax')},
    **{n: 'training.augmentation' for n in ('cutmix', 'mixup', 'random_crop')},
    **{n: 'training.data' for n in ('TensorDataset', 'default_collate')},
    **{n: 'training.extras' for n in ('DPSGD', 'RDPAccountant', 'SearchSpace', 'checkpoint', 'distillation_loss', 'grid_search', 'random_search')},
    **{n: 'training.schedulers' for n in ('LRScheduler', 'ReduceLROnPlateau')},
    **{n: 'utils.net' for n in ('Topology',)},
    **{n: 'utils.observability' for n in ('CompositeTracker', 'MLflowTracker', 'MemoryTracker', 'Timer', 'WandbTracker', 'estimate_flops', 'timeit')},
    **{n: 'utils.registry' for n in ('AIGateway', 'EvalMonitor')},
    # observability
    **{n: "utils.observability" for n in ("Profiler", "ExperimentTracker", "Logger")},
}

__all__ = sorted(_WHERE)


def __getattr__(name):
    where = _WHERE.get(name)
    if where is None:
        # everything else with a counterpart is collected in sneppx_alg_b200.compat_classes, .compat and .compat_services
        for mod in ("compat_classes", "compat", "compat_services"):
            try:
                obj = getattr(importlib.import_module(f"sneppx_alg_b200.{mod}"), name)
            except (AttributeError, ModuleNotFoundError):
                continue
            globals()[name] = obj
            return obj
        raise AttributeError(f"module 'SneppX_ALG' has no attribute '{name}'")
    obj = getattr(importlib.import_module(f"sneppx_alg_b200.{where}"), name)
    globals()[name] = obj
    return obj


def __dir__():
    return __all__
