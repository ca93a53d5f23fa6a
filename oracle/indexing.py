"""ctypes loader for oracle/indexing.c plus the same rule in pure Python (TEST
INFRASTRUCTURE ONLY).  The Python form follows tests/pipeline.py:10-15,75-78."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "_build" / "liboracle_indexing.so"
_MASK = (1 << 64) - 1


def hash_u64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def endpoint(seed, step, batch, sequence, context, size, world=1, rank=0) -> int:
    lo = max(8, context)
    key = (seed + step * batch * world + rank * batch + sequence) & _MASK
    return lo + hash_u64(key) % (size - lo)


def byte_batch(data: np.ndarray, seed, step, batch, context, world=1, rank=0):
    ends = [endpoint(seed, step, batch, s, context, len(data), world, rank) for s in range(batch)]
    x = np.stack([data[e - context:e] for e in ends])
    y = np.stack([data[e - context + 1:e + 1] for e in ends])
    return x, y


def build() -> Path:
    _LIB.parent.mkdir(exist_ok=True)
    src = _HERE / "indexing.c"
    if not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["gcc", "-O2", "-shared", "-fPIC", "-o", str(_LIB), str(src)])
    return _LIB


def load():
    lib = C.CDLL(str(build()))
    lib.oracle_hash_u64.restype = C.c_uint64
    lib.oracle_hash_u64.argtypes = [C.c_uint64]
    lib.oracle_endpoint.restype = C.c_int64
    lib.oracle_endpoint.argtypes = [C.c_uint64, C.c_uint64, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_int, C.c_int64]
    lib.oracle_byte_batch.restype = None
    lib.oracle_byte_batch.argtypes = [C.c_void_p, C.c_int64, C.c_uint64, C.c_uint64, C.c_int, C.c_int,
                                      C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    return lib


def byte_batch_c(data: np.ndarray, seed, step, batch, context, world=1, rank=0):
    lib = load()
    data = np.ascontiguousarray(data, dtype=np.uint8)
    x = np.empty((batch, context), np.uint8)
    y = np.empty((batch, context), np.uint8)
    lib.oracle_byte_batch(data.ctypes.data, len(data), seed, step, batch, world, rank, context,
                          x.ctypes.data, y.ctypes.data)
    return x, y
