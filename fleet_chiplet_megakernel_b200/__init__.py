"""B200-native persistent decode megakernel behind the MPK operator API.

``PersistentKernel`` mirrors python/mirage/mpk/persistent_kernel.py of the
reference for the decode path: the same constructor, layer methods, compile,
call and finalize.  It records the layers and drives the native runtime
(libb200mk.so, include/b200mk.h) through ctypes; torch is only used for
device tensors and streams at this edge.
"""
from .persistent_kernel import (PersistentKernel, DTensor, bfloat16, float16, float32, int32, int64, uint64,
                                valid_persistent_kernel_modes, get_configurations_from_gpu)
from .qwen3_graph import Qwen3Geometry, build_qwen3_graph, Qwen3Decoder, shard_qwen3_weights
from . import dsl, fleet
from .mpk import MPK, MPKMetadata, MirageModelConfig
from .qwen3_moe_graph import Qwen3MoeGeometry, build_qwen3_moe_graph, Qwen3MoeDecoder

__all__ = ["PersistentKernel", "DTensor", "bfloat16", "float16", "float32", "int32", "int64", "uint64",
           "valid_persistent_kernel_modes", "get_configurations_from_gpu", "Qwen3Geometry", "build_qwen3_graph",
           "Qwen3Decoder", "shard_qwen3_weights", "dsl", "fleet", "MPK", "MPKMetadata", "MirageModelConfig", "Qwen3MoeGeometry", "build_qwen3_moe_graph",
           "Qwen3MoeDecoder"]
