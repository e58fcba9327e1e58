"""tiga (B200-native build): drop-in ``import tiga as tg`` for the fused CSR
message-passing path of walkerchi/TIGA-lang, backed by hand-written sm_100a
CUDA kernels behind a C ABI (include/tiga_b200.h).

Public names follow python/tiga/__init__.py:45-105 of the reference for the
part of the API that lies on this path: ``MessagePassing``, ``Graph``, the
reducers, ``tg.math``, and the distributed placement objects.
"""
from . import codegen, control, math
from .control import repeat
from .program import GraphProgram, ProgramValue, program
from .distributed import ByDestination, DeviceMesh, GraphPlacement, HaloMap, derive_halo_map
from .graph import Graph, GraphSchema
from .kernel import AnalysisFinding, CompiledVariant, Kernel
from .message_passing import MessagePassing
from .ops import linear
from .storage import load, save
from .reducer import (MaxReducer, MeanReducer, OnlineSoftmaxItem, OnlineSoftmaxReducer, ProductReducer, Reducer,
                      ReducerCall, SumReducer, max, mean, online_softmax, prod, sum)

__version__ = "0.1.0"

__all__ = [
    "AnalysisFinding", "ByDestination", "CompiledVariant", "DeviceMesh", "Graph", "GraphPlacement",
    "GraphSchema", "HaloMap", "Kernel", "MaxReducer", "MeanReducer", "MessagePassing", "OnlineSoftmaxItem",
    "OnlineSoftmaxReducer", "ProductReducer", "Reducer", "ReducerCall", "SumReducer", "derive_halo_map",
    "GraphProgram", "ProgramValue", "codegen", "control", "linear", "load", "program", "repeat", "math", "max", "mean", "online_softmax", "prod", "save", "sum",
]
