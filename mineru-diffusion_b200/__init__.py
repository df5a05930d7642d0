"""B200-native block-diffusion decode path of MinerU-Diffusion's nano_dvlm engine.

The directory name carries a hyphen, so import it with
``importlib.import_module("mineru-diffusion_b200")``; after the first import the
alias ``mineru_diffusion_b200`` is registered too.
"""
import sys as _sys

from . import _lib, ops
from .decoder import DecoderEngine, DecoderWeights, LayerWeights
from .loader import load_decoder_weights
from .engine import (BlockManager, Config, Context, DecoderConfig, SamplingParams, Scheduler, Sequence,
                     SequenceStatus)
from .engine.llm_engine import LLMEngine
from .engine.model_runner import ModelRunner

_sys.modules.setdefault("mineru_diffusion_b200", _sys.modules[__name__])

__all__ = ["ops", "DecoderEngine", "DecoderWeights", "LayerWeights", "load_decoder_weights", "BlockManager", "Config", "Context",
           "DecoderConfig", "SamplingParams", "Scheduler", "Sequence", "SequenceStatus", "LLMEngine", "ModelRunner"]
