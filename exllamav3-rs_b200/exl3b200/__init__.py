"""Host-side mirror of the reference's op surface (src/ffi.rs) over libexl3b200.so."""
from .ffi import Checkpoint, Ctx, CudaGraph, Exl3Error, Linear, LinearLayer, Pool, lib, LIB_PATH, ROPE_NONE, ROPE_GPTJ, ROPE_NEOX  # noqa: F401
