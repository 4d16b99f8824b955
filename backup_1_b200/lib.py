"""ctypes binding of ``libdecxb.so`` (see ``include/decxb.h`` for the contract)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

GEMM_3XTF32, GEMM_1XTF32, GEMM_3XTF32_STRICT, GEMM_TF32_2XBF16 = 0, 1, 2, 3
GEMM_DEFAULT = GEMM_3XTF32_STRICT   # what the DECX-facing host layer uses unless told otherwise
TILE_AUTO, TILE_1CTA_128x128, TILE_2CTA_256x256, TILE_1CTA_128x256, TILE_1CTA_128x64 = 0, 1, 2, 3, 4
CONV_NO_COMPENSATE, CONV_ZERO_COMPENSATE = 0, 1
CONV_EXPLICIT, CONV_IMPLICIT = 0, 1
ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3

_PKG = Path(__file__).resolve().parent


class DecxbError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"decxb status {status}: {text}")
        self.status = status


def library_path() -> Path:
    """The CUDA library; DECXB_LIBRARY may name another build of it (the debug bounds build libdecxb_bounds.so)."""
    import os

    alt = os.environ.get("DECXB_LIBRARY")
    return Path(alt) if alt else _PKG / "libdecxb.so"


class ConvGeom(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("out_w", "out_h", "eq_w", "M", "Kp", "Np")]


class ArenaStats(C.Structure):
    _fields_ = [("bytes_in_use", C.c_size_t), ("bytes_cached", C.c_size_t), ("peak_bytes_in_use", C.c_size_t),
                ("n_driver_allocs", C.c_uint64), ("n_reuses", C.c_uint64)]


class Profile(C.Structure):
    _fields_ = [("ms", C.c_double * 4), ("launches", C.c_uint64 * 4)]

    def as_dict(self):
        names = ("gemm", "split", "pack", "fill")
        return {n: {"ms": self.ms[i], "launches": int(self.launches[i])} for i, n in enumerate(names)}


class TensorProbe(C.Structure):
    _fields_ = [("ms", C.c_double), ("tensor_tflops", C.c_double), ("algorithmic_tflops", C.c_double),
                ("iterations", C.c_int64), ("sms", C.c_int)]


_lib = None

# name -> (restype, argtypes); every symbol include/decxb.h declares
_i, _i64, _u64, _u32, _vp, _sz = C.c_int, C.c_int64, C.c_uint64, C.c_uint32, C.c_void_p, C.c_size_t
SIGNATURES = {
    "decxb_init": (_i, [_i, C.POINTER(_vp)]),
    "decxb_destroy": (_i, [_vp]),
    "decxb_status_string": (C.c_char_p, [_i]),
    "decxb_last_error": (C.c_char_p, [_vp]),
    "decxb_device": (_i, [_vp]),
    "decxb_stream": (_vp, [_vp]),
    "decxb_synchronize": (_i, [_vp]),
    "decxb_set_wait_limit_ms": (_i, [_vp, _i]),
    "decxb_malloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "decxb_free": (_i, [_vp, _vp]),
    "decxb_release_cached": (_i, [_vp]),
    "decxb_arena_get_stats": (_i, [_vp, C.POINTER(ArenaStats)]),
    "decxb_host_alloc": (_i, [_sz, C.POINTER(_vp)]),
    "decxb_host_free": (_i, [_vp]),
    "decxb_memcpy2d": (_i, [_vp, _vp, _sz, _vp, _sz, _sz, _sz, _i]),
    "decxb_memset": (_i, [_vp, _vp, _i, _sz]),
    "decxb_fill_uniform_f32": (_i, [_vp, _vp, _u64, _u64, _u64, _u32, _u64, _vp]),
    "decxb_gemm_f32": (_i, [_vp, _i, _i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "decxb_gemm_f32_act": (_i, [_vp, _i, _i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i, _vp, _i64, _vp]),
    "decxb_gemm_f32_nt": (_i, [_vp, _i, _i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "decxb_gemm_f32_host": (_i, [_vp, _i, _i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64]),
    "decxb_gemm_f16": (_i, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "decxb_gemm_f16_host": (_i, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64]),
    "decxb_gemm_f32_batched": (_i, [_vp, _i, _i, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp]),
    "decxb_gemm_f32_batched_host": (_i, [_vp, _i, _i, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64]),
    "decxb_gemm_f32_noalloc": (_i, [_i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, C.c_char_p, _sz]),
    "decxb_conv_geometry": (_i, [_i64, _i64, _i64, _i64, _i64, _i64, _i, C.POINTER(ConvGeom)]),
    "decxb_im2col_pack_f32": (_i, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _i, _vp, _i64, _i64, _i64, _vp]),
    "decxb_set_pack_variant": (_i, [_vp, _i]),
    "decxb_set_tile_group": (_i, [_vp, _i]),
    "decxb_set_tile_trace": (_i, [_vp, _vp, _i]),
    "decxb_set_wave_align": (_i, [_vp, _i]),
    "decxb_conv2_im2col_f32": (_i, [_vp, _i, _i, _i, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _vp]),
    "decxb_conv2_im2col_f32_act": (_i, [_vp, _i, _i, _i, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _i, _vp, _i64, _i64, _i64, _vp]),
    "decxb_conv2_im2col_f32_host": (_i, [_vp, _i, _i, _i, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64]),
    "decxb_shard_range": (_i, [_i64, _i, _i, C.POINTER(_i64), C.POINTER(_i64)]),
    "decxb_gemm_f32_rowshard": (_i, [_vp, _i, _i, _i, _i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp,
                                     C.POINTER(_i64), C.POINTER(_i64)]),
    "decxb_conv2_im2col_f32_batchshard": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _vp,
                                               _i64, _i64, _i64, _vp, C.POINTER(_i64), C.POINTER(_i64)]),
    "decxb_kernel_launch_count": (_u64, [_vp]),
    "decxb_selftest_bounded_wait": (_i, [_vp, _i]),
    "decxb_profile_enable": (_i, [_vp, _i]),
    "decxb_profile_read": (_i, [_vp, C.POINTER(Profile)]),
    "decxb_inject_pipeline_error": (_i, [_vp, _i]),
    "decxb_gemm_prepare_b": (_i, [_vp, _i, _i64, _i64, _vp, _i64, _vp, C.POINTER(_vp)]),
    "decxb_gemm_f32_prepared": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _i, _vp, _i64, _vp]),
    "decxb_gemm_release_b": (_i, [_vp, _vp, _vp]),
    "decxb_conv_prepare_filters": (_i, [_vp, _i, _i, _vp, _i64, _i64, _i64, _i64, _vp, C.POINTER(_vp)]),
    "decxb_conv2_im2col_f32_prepared": (_i, [_vp, _i, _vp, _i64, _i64, _vp, _vp, _i, _vp, _i64, _i64, _i64, _vp]),
    "decxb_conv_release_filters": (_i, [_vp, _vp, _vp]),
    "decxb_comm_unique_id": (_i, [_vp]),
    "decxb_comm_init": (_i, [_vp, _i, _i, _vp, _i, C.POINTER(_vp)]),
    "decxb_comm_destroy": (_i, [_vp]),
    "decxb_comm_last_error": (C.c_char_p, [_vp]),
    "decxb_comm_set_reserved_sms": (_i, [_vp, _i]),
    "decxb_comm_synchronize": (_i, [_vp]),
    "decxb_comm_allgather_blocks": (_i, [_vp, _vp, _sz, _i64, _vp]),
    "decxb_gemm_f32_rowshard_gather": (_i, [_vp, _vp, _i, _i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i, _vp]),
    "decxb_gemm_f32_rowshard_host": (_i, [_vp, _vp, _i, _i, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64]),
    "decxb_gemm_host_plan": (_i, [_i64, _i64, _i64, _i, _vp, _i]),
    "decxb_comm_selftest_handshake": (_i, [C.c_char_p, _i, _i, _vp, _i, C.c_char_p, _sz]),
    "decxb_probe_tensor_peak": (_i, [_vp, _i, C.c_double, C.POINTER(TensorProbe)]),
    "decxb_bounds_build": (_i, []),
    "decxb_selftest_bounds": (_i, [_vp]),
    "decxb_version": (C.c_char_p, []),
}


def load_library() -> C.CDLL:
    """Loads libdecxb.so and sets the prototypes.  Raises if the library is not built."""
    global _lib
    if _lib is None:
        p = library_path()
        if not p.exists():
            raise FileNotFoundError(f"{p} is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
                                    "or `make -C backup_1_b200/csrc`")
        L = C.CDLL(str(p))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Units [first, last) of `total` that `rank` of `world` owns (the library's partition rule)."""
    f, l = C.c_int64(0), C.c_int64(0)
    rc = load_library().decxb_shard_range(total, world, rank, C.byref(f), C.byref(l))
    if rc:
        raise DecxbError(rc, "bad world/rank")
    return f.value, l.value


def conv_geometry(W, H, depth, kW, kH, N, flag) -> ConvGeom:
    g = ConvGeom()
    rc = load_library().decxb_conv_geometry(W, H, depth, kW, kH, N, flag, C.byref(g))
    if rc:
        raise DecxbError(rc, load_library().decxb_status_string(rc).decode())
    return g


def _ptr(x):
    """Raw address of a torch tensor / numpy array / int / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(type(x))


class Context:
    """One decxb context (device, stream, arena).  Pointer arguments are torch tensors, numpy
    arrays or raw integer addresses; leading dimensions are in elements."""

    def __init__(self, device: int = 0):
        self.L = load_library()
        h = _vp()
        rc = self.L.decxb_init(device, C.byref(h))
        if rc:
            raise DecxbError(rc, self.L.decxb_status_string(rc).decode())
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.L.decxb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _chk(self, rc):
        if rc:
            raise DecxbError(rc, self.L.decxb_last_error(self.h).decode() or self.L.decxb_status_string(rc).decode())

    # -- runtime ------------------------------------------------------------------------
    def synchronize(self):
        self._chk(self.L.decxb_synchronize(self.h))

    def set_wait_limit_ms(self, ms: int):
        self._chk(self.L.decxb_set_wait_limit_ms(self.h, ms))

    def set_tile_group(self, tile_rows: int):
        self._chk(self.L.decxb_set_tile_group(self.h, tile_rows))

    def set_wave_align(self, mode: int):
        """0 off, 1 on (cooperative launches), 2 on with plain launches."""
        self._chk(self.L.decxb_set_wave_align(self.h, int(mode)))

    def launches(self) -> int:
        return int(self.L.decxb_kernel_launch_count(self.h))

    def profile_enable(self, on: bool = True):
        self._chk(self.L.decxb_profile_enable(self.h, 1 if on else 0))

    def profile_read(self) -> dict:
        p = Profile()
        self._chk(self.L.decxb_profile_read(self.h, C.byref(p)))
        return p.as_dict()

    def probe_tensor_peak(self, pattern: int, target_ms: float = 100.0) -> dict:
        """Tensor-core ceiling probe (see decxb_probe_tensor_peak)."""
        p = TensorProbe()
        self._chk(self.L.decxb_probe_tensor_peak(self.h, pattern, float(target_ms), C.byref(p)))
        return {"ms": p.ms, "tensor_tflops": p.tensor_tflops, "algorithmic_tflops": p.algorithmic_tflops,
                "iterations": int(p.iterations), "sms": p.sms}

    def malloc(self, nbytes: int) -> int:
        p = _vp()
        self._chk(self.L.decxb_malloc(self.h, nbytes, C.byref(p)))
        return p.value

    def free(self, ptr: int):
        self._chk(self.L.decxb_free(self.h, ptr))

    def release_cached(self):
        self._chk(self.L.decxb_release_cached(self.h))

    def arena_stats(self) -> ArenaStats:
        s = ArenaStats()
        self._chk(self.L.decxb_arena_get_stats(self.h, C.byref(s)))
        return s

    def fill_uniform(self, dst, rows, cols, pitch, seed, first_index=0, stream=None):
        self._chk(self.L.decxb_fill_uniform_f32(self.h, _ptr(dst), rows, cols, pitch, seed, first_index, stream))

    # -- GEMM ---------------------------------------------------------------------------
    def gemm(self, M, N, K, A, lda, B, ldb, D, ldd, Cin=None, ldc=0, mode=GEMM_DEFAULT, tile=TILE_AUTO, stream=None):
        self._chk(self.L.decxb_gemm_f32(self.h, mode, tile, M, N, K, _ptr(A), lda, _ptr(B), ldb,
                                        _ptr(Cin), ldc, _ptr(D), ldd, stream))

    def gemm_act(self, M, N, K, A, lda, B, ldb, D, ldd, Cin=None, ldc=0, bias=None, act=ACT_NONE,
                 mode=GEMM_DEFAULT, tile=TILE_AUTO, stream=None):
        self._chk(self.L.decxb_gemm_f32_act(self.h, mode, tile, M, N, K, _ptr(A), lda, _ptr(B), ldb, _ptr(Cin), ldc,
                                            _ptr(bias), act, _ptr(D), ldd, stream))

    def gemm_nt(self, M, N, K, A, lda, Bt, ldbt, D, ldd, Cin=None, ldc=0, mode=GEMM_DEFAULT, tile=TILE_AUTO, stream=None):
        self._chk(self.L.decxb_gemm_f32_nt(self.h, mode, tile, M, N, K, _ptr(A), lda, _ptr(Bt), ldbt,
                                           _ptr(Cin), ldc, _ptr(D), ldd, stream))

    def gemm_host(self, M, N, K, A, lda, B, ldb, D, ldd, Cin=None, ldc=0, mode=GEMM_DEFAULT, tile=TILE_AUTO):
        self._chk(self.L.decxb_gemm_f32_host(self.h, mode, tile, M, N, K, _ptr(A), lda, _ptr(B), ldb,
                                             _ptr(Cin), ldc, _ptr(D), ldd))

    def gemm_f16(self, M, N, K, A, lda, B, ldb, D, ldd, Cin=None, ldc=0, stream=None):
        self._chk(self.L.decxb_gemm_f16(self.h, M, N, K, _ptr(A), lda, _ptr(B), ldb, _ptr(Cin), ldc, _ptr(D), ldd, stream))

    def gemm_f16_host(self, M, N, K, A, lda, B, ldb, D, ldd, Cin=None, ldc=0):
        self._chk(self.L.decxb_gemm_f16_host(self.h, M, N, K, _ptr(A), lda, _ptr(B), ldb, _ptr(Cin), ldc, _ptr(D), ldd))

    def gemm_batched(self, batch, M, N, K, A, lda, sA, B, ldb, sB, D, ldd, sD, Cin=None, ldc=0, sC=0,
                     mode=GEMM_DEFAULT, tile=TILE_AUTO, stream=None):
        self._chk(self.L.decxb_gemm_f32_batched(self.h, mode, tile, batch, M, N, K, _ptr(A), lda, sA, _ptr(B), ldb, sB,
                                                _ptr(Cin), ldc, sC, _ptr(D), ldd, sD, stream))

    def gemm_batched_host(self, batch, M, N, K, A, lda, sA, B, ldb, sB, D, ldd, sD, Cin=None, ldc=0, sC=0,
                          mode=GEMM_DEFAULT, tile=TILE_AUTO):
        self._chk(self.L.decxb_gemm_f32_batched_host(self.h, mode, tile, batch, M, N, K, _ptr(A), lda, sA, _ptr(B), ldb, sB,
                                                     _ptr(Cin), ldc, sC, _ptr(D), ldd, sD))

    def prepare_b(self, K, N, B, ldb, mode=GEMM_DEFAULT, stream=None) -> int:
        """Splits and transposes B once (decxb_gemm_prepare_b); returns the handle."""
        h = _vp()
        self._chk(self.L.decxb_gemm_prepare_b(self.h, mode, K, N, _ptr(B), ldb, stream, C.byref(h)))
        return h.value

    def gemm_prepared(self, M, A, lda, pb, D, ldd, Cin=None, ldc=0, bias=None, act=ACT_NONE, tile=TILE_AUTO, stream=None):
        self._chk(self.L.decxb_gemm_f32_prepared(self.h, tile, M, _ptr(A), lda, pb, _ptr(Cin), ldc, _ptr(bias), act,
                                                 _ptr(D), ldd, stream))

    def release_b(self, pb, stream=None):
        self._chk(self.L.decxb_gemm_release_b(self.h, pb, stream))

    # -- convolution ----------------------------------------------------------------------
    def set_pack_variant(self, variant: int):
        self._chk(self.L.decxb_set_pack_variant(self.h, variant))

    def im2col_pack(self, src, W, H, depth, kW, kH, flag, i2c, batch=1, src_stride=0, i2c_stride=0, stream=None):
        self._chk(self.L.decxb_im2col_pack_f32(self.h, _ptr(src), W, H, depth, kW, kH, flag, _ptr(i2c),
                                               batch, src_stride, i2c_stride, stream))

    def conv2_im2col(self, src, W, H, depth, filters, kW, kH, N, dst, flag=CONV_ZERO_COMPENSATE, batch=1,
                     src_stride=0, dst_stride=0, mode=GEMM_DEFAULT, algo=CONV_EXPLICIT, stream=None):
        self._chk(self.L.decxb_conv2_im2col_f32(self.h, mode, algo, flag, _ptr(src), W, H, depth, _ptr(filters),
                                                kW, kH, N, _ptr(dst), batch, src_stride, dst_stride, stream))

    def conv_prepare_filters(self, filters, kW, kH, depth, N, mode=GEMM_DEFAULT, algo=CONV_IMPLICIT, stream=None) -> int:
        h = _vp()
        self._chk(self.L.decxb_conv_prepare_filters(self.h, mode, algo, _ptr(filters), kW, kH, depth, N, stream, C.byref(h)))
        return h.value

    def conv2_im2col_prepared(self, src, W, H, pf, dst, flag=CONV_ZERO_COMPENSATE, batch=1, src_stride=0, dst_stride=0,
                              bias=None, act=ACT_NONE, stream=None):
        self._chk(self.L.decxb_conv2_im2col_f32_prepared(self.h, flag, _ptr(src), W, H, pf, _ptr(bias), act, _ptr(dst),
                                                         batch, src_stride, dst_stride, stream))

    def conv_release_filters(self, pf, stream=None):
        self._chk(self.L.decxb_conv_release_filters(self.h, pf, stream))

    def gemm_rowshard(self, world, rank, M, N, K, A_rows, lda, B, ldb, D_rows, ldd, C_rows=None, ldc=0,
                      mode=GEMM_DEFAULT, tile=TILE_AUTO, stream=None):
        """This rank's rows of D = A B (+C); returns the row range [first, last) it computed."""
        f, l = C.c_int64(0), C.c_int64(0)
        self._chk(self.L.decxb_gemm_f32_rowshard(self.h, mode, tile, world, rank, M, N, K, _ptr(A_rows), lda, _ptr(B), ldb,
                                                 _ptr(C_rows), ldc, _ptr(D_rows), ldd, stream, C.byref(f), C.byref(l)))
        return f.value, l.value

    def conv2_im2col_batchshard(self, world, rank, src, W, H, depth, filters, kW, kH, N, dst, batch,
                                flag=CONV_ZERO_COMPENSATE, src_stride=0, dst_stride=0, mode=GEMM_DEFAULT,
                                algo=CONV_IMPLICIT, stream=None):
        """This rank's images of the batch; src/dst point at its first image.  Returns [first, last)."""
        f, l = C.c_int64(0), C.c_int64(0)
        self._chk(self.L.decxb_conv2_im2col_f32_batchshard(self.h, mode, algo, flag, world, rank, _ptr(src), W, H, depth,
                                                           _ptr(filters), kW, kH, N, _ptr(dst), batch, src_stride,
                                                           dst_stride, stream, C.byref(f), C.byref(l)))
        return f.value, l.value

    def conv2_im2col_act(self, src, W, H, depth, filters, kW, kH, N, dst, bias=None, act=ACT_NONE,
                         flag=CONV_ZERO_COMPENSATE, batch=1, src_stride=0, dst_stride=0, mode=GEMM_DEFAULT,
                         algo=CONV_IMPLICIT, stream=None):
        self._chk(self.L.decxb_conv2_im2col_f32_act(self.h, mode, algo, flag, _ptr(src), W, H, depth, _ptr(filters),
                                                    kW, kH, N, _ptr(bias), act, _ptr(dst), batch, src_stride,
                                                    dst_stride, stream))

    def conv2_im2col_host(self, src, W, H, depth, filters, kW, kH, N, dst, flag=CONV_ZERO_COMPENSATE, batch=1,
                          src_stride=0, dst_stride=0, mode=GEMM_DEFAULT, algo=CONV_EXPLICIT):
        self._chk(self.L.decxb_conv2_im2col_f32_host(self.h, mode, algo, flag, _ptr(src), W, H, depth, _ptr(filters),
                                                     kW, kH, N, _ptr(dst), batch, src_stride, dst_stride))


def _order_after_torch(fn):
    """Device-resident entries called WITHOUT an explicit stream run on the context's own stream, which is not ordered
    with torch's streams: if any argument is a torch CUDA tensor, wait for torch's current stream first, so that a
    fill or copy torch has queued (a NaN sentinel, an upload) is complete before the library touches the tensor."""
    import functools

    @functools.wraps(fn)
    def wrapper(self, *args, **kwargs):
        if kwargs.get("stream") is None:
            for a in list(args) + list(kwargs.values()):
                if getattr(a, "is_cuda", False):
                    import torch

                    torch.cuda.current_stream(a.device).synchronize()
                    break
        return fn(self, *args, **kwargs)
    return wrapper


for _name in ("fill_uniform", "gemm", "gemm_act", "gemm_nt", "gemm_f16", "gemm_batched", "prepare_b", "gemm_prepared",
              "im2col_pack", "conv2_im2col", "conv2_im2col_act", "conv2_im2col_prepared", "conv_prepare_filters",
              "gemm_rowshard", "conv2_im2col_batchshard"):
    setattr(Context, _name, _order_after_torch(getattr(Context, _name)))


class Comm:
    """A communicator over NCCL for gathering the blocks of a sharded result (decxb_comm_*).
    Rank 0 makes the id with Comm.unique_id() and hands the 128 bytes to the other ranks."""

    def __init__(self, ctx: Context, world: int, rank: int, uid: bytes, timeout_ms: int = 30000):
        self.ctx, self.L = ctx, ctx.L
        h = _vp()
        buf = C.create_string_buffer(bytes(uid), 128)
        rc = self.L.decxb_comm_init(ctx.h, world, rank, buf, timeout_ms, C.byref(h))
        if rc:
            raise DecxbError(rc, self.L.decxb_last_error(ctx.h).decode() or self.L.decxb_status_string(rc).decode())
        self.h, self.world, self.rank = h, world, rank

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        rc = load_library().decxb_comm_unique_id(buf)
        if rc:
            raise DecxbError(rc, "decxb_comm_unique_id (is libnccl.so.2 loadable?)")
        return buf.raw

    def _chk(self, rc):
        if rc:
            raise DecxbError(rc, self.L.decxb_comm_last_error(self.h).decode() or self.L.decxb_status_string(rc).decode())

    def set_reserved_sms(self, sms: int):
        self._chk(self.L.decxb_comm_set_reserved_sms(self.h, sms))

    def synchronize(self):
        self._chk(self.L.decxb_comm_synchronize(self.h))

    def allgather_blocks(self, base, unit_bytes: int, total_units: int, stream=None):
        if stream is None and getattr(base, "is_cuda", False):
            import torch

            torch.cuda.current_stream(base.device).synchronize()
        self._chk(self.L.decxb_comm_allgather_blocks(self.h, _ptr(base), unit_bytes, total_units, stream))

    def gemm_rowshard_gather(self, M, N, K, A_rows, lda, B, ldb, D_full, groups=4, mode=GEMM_DEFAULT, tile=TILE_AUTO, stream=None):
        if stream is None and getattr(D_full, "is_cuda", False):
            import torch

            torch.cuda.current_stream(D_full.device).synchronize()
        self._chk(self.L.decxb_gemm_f32_rowshard_gather(self.ctx.h, self.h, mode, tile, M, N, K, _ptr(A_rows), lda, _ptr(B), ldb,
                                                        _ptr(D_full), groups, stream))

    def gemm_rowshard_host(self, M, N, K, hA_rows, lda, hB, ldb, hD_rows, ldd, mode=GEMM_DEFAULT, tile=TILE_AUTO):
        """Host-resident operands: this rank's rows of D; B is uploaded in shares and all-gathered on the device."""
        self._chk(self.L.decxb_gemm_f32_rowshard_host(self.ctx.h, self.h, mode, tile, M, N, K, _ptr(hA_rows), lda, _ptr(hB), ldb,
                                                      _ptr(hD_rows), ldd))

    def close(self):
        if getattr(self, "h", None):
            self.L.decxb_comm_destroy(self.h)
            self.h = None
