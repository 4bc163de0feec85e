"""Parts a model is assembled from: mixers, feed-forwards, norms, position encodings, blocks."""
from .base import (CacheView, FeedForward, Mixer, Norm, NormedStream, PagedBuffer, PagedSpec, PostNormed, ScaledPair, StreamState, Part, PositionEncoding, StateSpec,
                   TensorSpec, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, make_part,
                   register_feed_forward, register_mixer, register_norm, register_position_encoding)
from .norm import LayerNorm, NoNorm, RMSNorm
from .rope import RotaryEncoding, ScaledRotaryEncoding
from .attention import GQAttention
from .shortconv import ShortConv
from .recurrent import GatedDeltaMixer, Mamba2Mixer, RGLRUMixer
from .feedforward import SwiGLU
from .moe import SparseMoE
from .embedding import OutputHead, TokenEmbedding
from .block import BLOCKS, ParallelBlock, PreNormBlock, SandwichBlock, register_block
from .latent import LatentAttention
from .loop import StreamInjection
from .hyper import HyperBlock, HyperPending
from .parallel import ParallelMixer
from .linear_memory import GatedLinearAttentionMixer, MatrixMemoryMixer

__all__ = [
    "CacheView", "FeedForward", "Mixer", "Norm", "NormedStream", "PagedBuffer", "PagedSpec", "StreamState", "Part", "PositionEncoding", "StateSpec",
    "TensorSpec", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "BLOCKS", "make_part",
    "register_feed_forward", "register_mixer", "register_norm", "register_position_encoding",
    "register_block", "RMSNorm", "RotaryEncoding", "GQAttention", "ShortConv", "SwiGLU", "OutputHead",
    "TokenEmbedding", "PreNormBlock", "SandwichBlock", "PostNormed", "ScaledRotaryEncoding", "GatedDeltaMixer", "Mamba2Mixer",
    "LayerNorm", "RGLRUMixer", "SparseMoE", "HyperBlock", "HyperPending", "ParallelMixer",
    "NoNorm", "MatrixMemoryMixer", "GatedLinearAttentionMixer", "ParallelBlock", "ScaledPair", "LatentAttention", "StreamInjection",
]
