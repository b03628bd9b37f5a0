from .base import Part, StepContext, StepPlan, to_device_matrix, to_device_vector
from .linear import linear
from .norm import RMSNorm
from .rotary import RotaryTable
from .attention import Mixer, GQAAttention
from .feedforward import FeedForward, SwiGLU
from .block import PreNormBlock
from .embedding import Embedding, OutputHead
from .model import DecoderModel, LayerCall

__all__ = ["Part", "StepContext", "StepPlan", "to_device_matrix", "to_device_vector", "linear", "RMSNorm",
           "RotaryTable", "Mixer", "GQAAttention", "FeedForward", "SwiGLU", "PreNormBlock",
           "Embedding", "OutputHead", "DecoderModel", "LayerCall"]
