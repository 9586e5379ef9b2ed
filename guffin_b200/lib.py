"""ctypes binding of libguffin_b200.so -- the same C ABI a C++/other-language host binds.

There is no CPU fallback: if the shared library is missing or a call fails, this raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libguffin_b200.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "guffin_b200.h")

Q8_0, Q4_K, Q6_K = 8, 12, 14
MAX_ROWS = 8

GF_OK, GF_ERR_INVALID, GF_ERR_STATE, GF_ERR_CUDA, GF_ERR_UNAVAILABLE, GF_ERR_NUMERIC, GF_ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6


class GuffinError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"guffin_b200 status {status}: {message}")
        self.status = status


_lib = None


def load() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m guffin_b200.build` "
                "(the CUDA extension is the only implementation; there is no CPU path)")
        _lib = C.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(L: C.CDLL) -> None:
    vp, u32, u64, i32, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_size_t
    L.gf_last_error.restype = C.c_char_p
    L.gf_version.restype = C.c_char_p
    sigs = {
        "gf_device_count": [C.POINTER(i32)],
        "gf_set_device": [i32],
        "gf_memory_info": [C.POINTER(sz), C.POINTER(sz)],
        "gf_malloc": [C.POINTER(vp), sz],
        "gf_free": [vp],
        "gf_host_alloc": [C.POINTER(vp), sz],
        "gf_host_free": [vp],
        "gf_memset": [vp, i32, sz, vp],
        "gf_upload": [vp, vp, sz, vp],
        "gf_download": [vp, vp, sz, vp],
        "gf_copy": [vp, vp, sz, vp],
        "gf_stream_create": [C.POINTER(vp)],
        "gf_stream_destroy": [vp],
        "gf_stream_synchronize": [vp],
        "gf_event_create": [C.POINTER(vp)],
        "gf_event_destroy": [vp],
        "gf_event_record": [vp, vp],
        "gf_event_synchronize": [vp],
        "gf_event_elapsed_ms": [vp, vp, C.POINTER(C.c_float)],
        "gf_pack_weight": [i32, vp, u64, u64, vp, vp],
        "gf_unpack_weight": [i32, vp, u64, u64, vp, vp],
        "gf_dequantize": [i32, vp, u64, vp, vp],
        "gf_quantize_f16_q8_0": [vp, u64, vp, vp, vp],
        "gf_requantize_q6_k_q4_k": [vp, u64, vp, vp, vp],
        "gf_matmul": [i32, vp, vp, vp, u32, u64, u64, vp, vp],
        "gf_matmul_check": [vp],
        "gf_matmul_host": [i32, vp, vp, vp, u32, u64, u64],
        "gf_matmul_static": [i32, vp, vp, vp, u32, u64, u64, vp],
        "gf_matmul_static_check": [vp],
        "gf_prefill_matmul": [i32, vp, vp, vp, u32, u64, u64, vp, vp],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = i32
    L.gf_packed_weight_bytes.argtypes = [i32, u64, u64]
    L.gf_packed_weight_bytes.restype = sz
    L.gf_matmul_workspace_bytes.argtypes = [i32, u32, u64, u64]
    L.gf_matmul_workspace_bytes.restype = sz
    L.gf_prefill_workspace_bytes.argtypes = [u64]
    L.gf_prefill_workspace_bytes.restype = sz
    L.gf_matmul_static_capacity.argtypes = []
    L.gf_matmul_static_capacity.restype = sz
    _apply(L, SIGNATURES)


def _apply(L: C.CDLL, signatures: dict) -> None:
    for name, (res, args) in signatures.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = res


# Signatures registered by the higher-level modules (model, engine).
SIGNATURES: dict = {}


def register(signatures: dict) -> None:
    SIGNATURES.update(signatures)
    if _lib is not None:
        _apply(_lib, signatures)


def check(status: int) -> None:
    if status != GF_OK:
        raise GuffinError(status, load().gf_last_error().decode())


def device_count() -> int:
    n = C.c_int(0)
    status = load().gf_device_count(C.byref(n))
    return n.value if status == GF_OK else 0


class Event:
    """A device timestamp on a stream (gf_event_*)."""

    def __init__(self):
        ptr = C.c_void_p()
        check(load().gf_event_create(C.byref(ptr)))
        self.ptr = ptr.value

    def record(self, stream=None):
        check(load().gf_event_record(self.ptr, stream))

    def synchronize(self):
        check(load().gf_event_synchronize(self.ptr))

    def elapsed_ms(self, end: "Event") -> float:
        ms = C.c_float()
        check(load().gf_event_elapsed_ms(self.ptr, end.ptr, C.byref(ms)))
        return ms.value


class DeviceBuffer:
    """A device allocation owned through the C ABI (gf_malloc / gf_free)."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        ptr = C.c_void_p()
        check(load().gf_malloc(C.byref(ptr), self.nbytes))
        self.ptr = ptr.value

    @classmethod
    def from_numpy(cls, array: np.ndarray, stream=None) -> "DeviceBuffer":
        array = np.ascontiguousarray(array)
        buf = cls(array.nbytes)
        buf.upload(array, stream)
        return buf

    def upload(self, array: np.ndarray, stream=None) -> None:
        array = np.ascontiguousarray(array)
        assert array.nbytes <= self.nbytes
        check(load().gf_upload(self.ptr, array.ctypes.data, array.nbytes, stream))
        check(load().gf_stream_synchronize(stream))

    def download(self, dtype, count: int | None = None, stream=None) -> np.ndarray:
        dtype = np.dtype(dtype)
        count = self.nbytes // dtype.itemsize if count is None else count
        out = np.empty(count, dtype)
        check(load().gf_download(out.ctypes.data, self.ptr, out.nbytes, stream))
        check(load().gf_stream_synchronize(stream))
        return out

    def zero(self, stream=None) -> None:
        check(load().gf_memset(self.ptr, 0, self.nbytes, stream))

    def free(self) -> None:
        if getattr(self, "ptr", None):
            load().gf_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PackedWeight:
    """A [K, N] quantised matrix resident in the streaming layout."""

    def __init__(self, dtype: int, k: int, n: int, native: np.ndarray | None = None, keep_native: bool = False):
        L = load()
        self.dtype, self.k, self.n = dtype, k, n
        self.nbytes = L.gf_packed_weight_bytes(dtype, k, n)
        if self.nbytes == 0:
            raise GuffinError(GF_ERR_INVALID, L.gf_last_error().decode())
        self.packed = DeviceBuffer(self.nbytes)
        self.native = None
        if native is not None:
            staging = DeviceBuffer.from_numpy(np.ascontiguousarray(native, np.uint8))
            check(L.gf_pack_weight(dtype, staging.ptr, k, n, self.packed.ptr, None))
            check(L.gf_stream_synchronize(None))
            if keep_native:
                self.native = staging
            else:
                staging.free()

    def unpack(self) -> np.ndarray:
        from .synthetic import weight_bytes
        L = load()
        out = DeviceBuffer(weight_bytes(self.dtype, self.k, self.n))
        check(L.gf_unpack_weight(self.dtype, self.packed.ptr, self.k, self.n, out.ptr, None))
        result = out.download(np.uint8)
        out.free()
        return result


def dequantize(dtype: int, native: np.ndarray) -> np.ndarray:
    from .synthetic import BLOCK_BYTES, BLOCK_ELEMENTS
    L = load()
    native = np.ascontiguousarray(native, np.uint8).reshape(-1)
    blocks = native.size // BLOCK_BYTES[dtype]
    src = DeviceBuffer.from_numpy(native)
    dst = DeviceBuffer(blocks * BLOCK_ELEMENTS[dtype] * 4)
    check(L.gf_dequantize(dtype, src.ptr, blocks, dst.ptr, None))
    out = dst.download(np.float32)
    src.free()
    dst.free()
    return out


def quantize_f16_q8_0(f16_bits: np.ndarray):
    """Binary16 values (uint16 bits, a multiple of 32) -> (status word, Q8_0 blocks) on the device."""
    L = load()
    f16_bits = np.ascontiguousarray(f16_bits, np.uint16).reshape(-1)
    blocks = f16_bits.size // 32
    src, dst, flag = DeviceBuffer.from_numpy(f16_bits), DeviceBuffer(blocks * 34), DeviceBuffer(16)
    flag.zero()
    check(L.gf_quantize_f16_q8_0(src.ptr, blocks, dst.ptr, flag.ptr, None))
    out, status = dst.download(np.uint8), int(flag.download(np.uint32)[0])
    for b in (src, dst, flag):
        b.free()
    return status, out


def requantize_q6k_q4k(q6k: np.ndarray):
    """Q6_K blocks -> (status word, Q4_K blocks) on the device, block for block."""
    L = load()
    q6k = np.ascontiguousarray(q6k, np.uint8).reshape(-1)
    blocks = q6k.size // 210
    src, dst, flag = DeviceBuffer.from_numpy(q6k), DeviceBuffer(blocks * 144), DeviceBuffer(16)
    flag.zero()
    check(L.gf_requantize_q6_k_q4_k(src.ptr, blocks, dst.ptr, flag.ptr, None))
    out, status = dst.download(np.uint8), int(flag.download(np.uint32)[0])
    for b in (src, dst, flag):
        b.free()
    return status, out


def matmul(weight: PackedWeight, x: np.ndarray) -> np.ndarray:
    """y = x @ deq(W)^T on the GPU with device-resident staging (x uploaded, y downloaded)."""
    L = load()
    x = np.ascontiguousarray(x, np.float32).reshape(-1, weight.k)
    rows = x.shape[0]
    xd = DeviceBuffer.from_numpy(x)
    yd = DeviceBuffer(rows * weight.n * 4)
    ws_bytes = L.gf_matmul_workspace_bytes(weight.dtype, rows, weight.k, weight.n)
    ws = DeviceBuffer(ws_bytes) if ws_bytes else None
    check(L.gf_matmul(weight.dtype, weight.packed.ptr, xd.ptr, yd.ptr, rows, weight.k, weight.n,
                      ws.ptr if ws else None, None))
    check(L.gf_matmul_check(None))
    y = yd.download(np.float32).reshape(rows, weight.n)
    for b in (xd, yd, ws):
        if b:
            b.free()
    return y


def prefill_matmul(weight: PackedWeight, x: np.ndarray) -> np.ndarray:
    """y = x @ deq(W)^T for up to 256 rows on the tensor cores (bf16 operands, f32 accumulation); the
    result has 128 or 256 rows (whole halves), rows beyond the live ones zero."""
    L = load()
    x = np.ascontiguousarray(x, np.float32).reshape(-1, weight.k)
    rows = x.shape[0]
    xd = DeviceBuffer.from_numpy(x)
    padded = (rows + 127) // 128 * 128
    yd = DeviceBuffer(padded * weight.n * 4)
    ws = DeviceBuffer(L.gf_prefill_workspace_bytes(weight.k))
    check(L.gf_prefill_matmul(weight.dtype, weight.packed.ptr, xd.ptr, yd.ptr, rows, weight.k, weight.n, ws.ptr, None))
    y = yd.download(np.float32).reshape(padded, weight.n)
    for b in (xd, yd, ws):
        b.free()
    return y


def matmul_host(weight: PackedWeight, x: np.ndarray) -> np.ndarray:
    """The host-buffer entry point (gf_matmul_host): what a host engine calls per projection."""
    L = load()
    x = np.ascontiguousarray(x, np.float32).reshape(-1, weight.k)
    y = np.empty((x.shape[0], weight.n), np.float32)
    check(L.gf_matmul_host(weight.dtype, weight.packed.ptr, x.ctypes.data, y.ctypes.data, x.shape[0],
                           weight.k, weight.n))
    return y
