"""citlali_b200: a small generation library for the Qwen3 dense decoder on one B200.

    import citlali_b200 as cb
    session = cb.InferenceSession().load_model("model_dir", max_context=2048)
    results = session.generate([[1, 2, 3], [4, 5]], cb.GenerationOptions(max_new_tokens=16))
"""
from .errors import CitlaliError, require
from .config import (QwenConfig, ModelSpec, LayerSpec, PartSpec, ScheduleStep, config_from_dict,
                     config_from_model_dir, register_architecture, registered_architectures,
                     unregister_architecture)
from .weights import (SafetensorsFile, TensorSpec, WeightHandle, WeightLoader, write_random_model,
                      write_safetensors)
from .cache import PAGE_SIZE, KVRequirement, SequenceCache, StateRequirement
from .parts import BuildContext, StepBatch, build_part, register_part, registered_parts, unregister_part
from .engine import (DecoderModel, GenerationOptions, GenerationResult, InferenceSession, StepEntry,
                     StopReason, expected_tensors, run_generation)
from .sampling import Sampler, uniform

__all__ = [n for n in dir() if not n.startswith("_")]
