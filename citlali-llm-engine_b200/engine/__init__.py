from .generate import GenerationOptions, GenerationResult, StopReason, run_generation
from .model import DecoderModel, expected_tensors
from .session import InferenceSession, parse_dtype
from .step import StepEntry, pack_step
