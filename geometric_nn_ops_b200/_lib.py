"""ctypes binding of libtri_b200.so (declarations in include/tri_b200.h).

The library is built in-tree by ``geometric_nn_ops_b200.build``.  There is no
fallback: if it is missing, or a call fails, a ``RuntimeError`` is raised.
"""

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_longlong, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TRI_B200_LIB", os.path.join(_HERE, "libtri_b200.so"))

F32, BF16, F16 = 0, 1, 2
ERR_UNSUPPORTED = -3   # TRI_ERR_UNSUPPORTED
PREC_IEEE, PREC_TF32 = 0, 1
OUTGOING, INCOMING = 0, 1


class TriAttnDesc(Structure):
    _fields_ = [
        ("B", c_int32), ("n_seq", c_int32), ("n_res", c_int32), ("H", c_int32), ("D", c_int32),
        ("dtype", c_int32), ("precision", c_int32), ("scale", c_float),
        ("q_st", c_int64 * 4), ("k_st", c_int64 * 4), ("v_st", c_int64 * 4), ("o_st", c_int64 * 4),
        ("do_st", c_int64 * 4), ("dq_st", c_int64 * 4), ("dk_st", c_int64 * 4), ("dv_st", c_int64 * 4),
        ("bias_st", c_int64 * 3), ("mask_st", c_int64 * 2),
    ]


class TriMulDesc(Structure):
    _fields_ = [
        ("B", c_int32), ("N", c_int32), ("C", c_int32), ("Ch", c_int32),
        ("dtype", c_int32), ("precision", c_int32), ("direction", c_int32), ("eps", c_float),
    ]


class TriAttnProjDesc(Structure):
    _fields_ = [("M", c_int64), ("C", c_int32), ("H", c_int32), ("D", c_int32), ("dtype", c_int32), ("precision", c_int32),
                ("eps", c_float)]


class TriGemmDesc(Structure):
    _fields_ = [
        ("M", c_int32), ("N", c_int32), ("K", c_int32), ("batch", c_int32), ("dtype", c_int32),
        ("a_mn_major", c_int32), ("b_mn_major", c_int32), ("out_f32", c_int32),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("batch_a", c_int64), ("batch_b", c_int64), ("batch_c", c_int64),
    ]


WEIGHT_NAMES = (
    "norm_in_weight", "norm_in_bias", "p_in_weight", "p_in_bias", "g_in_weight", "g_in_bias",
    "norm_out_weight", "norm_out_bias", "p_out_weight", "p_out_bias", "g_out_weight", "g_out_bias",
)
_ABI_FIELD = {n: n.replace("_weight", "_w").replace("_bias", "_b") for n in WEIGHT_NAMES}


class TriMulWeights(Structure):
    _fields_ = [(_ABI_FIELD[n], c_void_p) for n in WEIGHT_NAMES]


class TriMulWeightGrads(Structure):
    _fields_ = [(_ABI_FIELD[n], c_void_p) for n in WEIGHT_NAMES]


class TriMulShardDesc(Structure):
    _fields_ = [
        ("B", c_int32), ("rows", c_int32), ("N", c_int32), ("C", c_int32), ("Ch", c_int32),
        ("dtype", c_int32), ("precision", c_int32), ("eps", c_float),
    ]


class TriMulShardBufs(Structure):
    _fields_ = [
        ("x", c_void_p), ("mask", c_void_p), ("w", POINTER(TriMulWeights)), ("saved", c_void_p),
        ("a_cm", c_void_p), ("b_cm", c_void_p), ("t_cm", c_void_p), ("out", c_void_p),
        ("d_out", c_void_p), ("dt_cm", c_void_p), ("dx", c_void_p), ("g", POINTER(TriMulWeightGrads)),
        ("peer_ab", POINTER(c_void_p)), ("peer_world", ctypes.c_int32), ("peer_rank", ctypes.c_int32),
        ("prep", c_void_p), ("prep_ready", ctypes.c_int32),
    ]


PHASE_PROJECT, PHASE_OUTPUT, PHASE_OUTPUT_BWD, PHASE_PROJECT_BWD = 0, 1, 2, 3

class TriScatterDesc(ctypes.Structure):
    _fields_ = [("dims", ctypes.c_int64 * 3), ("dst_stride", ctypes.c_int64 * 3), ("dst_base_run", ctypes.c_int64),
                ("run_bytes", ctypes.c_int64), ("peer_dim", ctypes.c_int32), ("n_peers", ctypes.c_int32)]


class TriPeerSignal(ctypes.Structure):
    _fields_ = [("flag_ptrs", POINTER(c_void_p)), ("state", c_void_p), ("rank", ctypes.c_int32), ("n_peers", ctypes.c_int32)]


EXPORTS = {
    "tri_abi_version": (c_int, []),
    "tri_last_error": (c_char_p, []),
    "tri_last_path": (c_char_p, []),
    "tri_launch_count": (c_longlong, []),
    "tri_reset_launch_count": (None, []),
    "tri_profile_enable": (None, [c_int]),
    "tri_profile_summary": (c_int, [ctypes.c_char_p, c_size_t]),
    "tri_attn_ws_bytes": (c_size_t, [POINTER(TriAttnDesc), c_int]),
    "tri_attn_fwd": (c_int, [POINTER(TriAttnDesc)] + [c_void_p] * 8 + [c_size_t, c_void_p]),
    "tri_attn_bwd": (c_int, [POINTER(TriAttnDesc)] + [c_void_p] * 13 + [c_size_t, c_void_p]),
    "tri_attn_bwd_noalloc": (c_int, [POINTER(TriAttnDesc)] + [c_void_p] * 12 + [c_void_p]),
    "tri_attn_project_ws_bytes": (c_size_t, [POINTER(TriAttnProjDesc)]),
    "tri_attn_project": (c_int, [POINTER(TriAttnProjDesc)] + [c_void_p] * 8 + [c_size_t, c_void_p]),
    "tri_mul_saved_bytes": (c_size_t, [POINTER(TriMulDesc)]),
    "tri_mul_ws_bytes": (c_size_t, [POINTER(TriMulDesc), c_int]),
    "tri_mul_fwd": (c_int, [POINTER(TriMulDesc), c_void_p, c_void_p, POINTER(TriMulWeights), c_void_p, c_void_p,
                            c_void_p, c_size_t, c_void_p]),
    "tri_mul_bwd": (c_int, [POINTER(TriMulDesc), c_void_p, c_void_p, POINTER(TriMulWeights), c_void_p, c_void_p,
                            c_void_p, POINTER(TriMulWeightGrads), c_void_p, c_size_t, c_void_p]),
    "tri_mul_shard_saved_bytes": (c_size_t, [POINTER(TriMulShardDesc)]),
    "tri_mul_shard_ws_bytes": (c_size_t, [POINTER(TriMulShardDesc), c_int]),
    "tri_mul_shard_prep_bytes": (c_size_t, [POINTER(TriMulShardDesc)]),
    "tri_mul_shard_phase": (c_int, [POINTER(TriMulShardDesc), c_int, POINTER(TriMulShardBufs), c_void_p, c_size_t,
                                    c_void_p]),
    "tri_bgemm": (c_int, [POINTER(TriGemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "tri_permute_runs": (c_int, [c_void_p, c_void_p, POINTER(ctypes.c_int64 * 3), POINTER(ctypes.c_int32 * 3),
                                 ctypes.c_int64, c_void_p]),
    "tri_scatter_runs": (c_int, [POINTER(TriScatterDesc), c_void_p, POINTER(c_void_p), c_void_p]),
    "tri_scatter_runs_dma": (c_int, [POINTER(TriScatterDesc), c_void_p, POINTER(c_void_p), c_void_p]),
    "tri_peer_barrier": (c_int, [POINTER(TriPeerSignal), c_int64, c_void_p]),
    "tri_ws_status": (c_int, [c_void_p, c_void_p]),
}

_lib = None


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m geometric_nn_ops_b200.build` "
                "(there is no fallback implementation)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().tri_last_error().decode(errors="replace")
        raise RuntimeError(f"{what} failed with code {code}: {msg}")


def check_device_status(ws, stream) -> None:
    """With TRI_B200_CHECK=1, read back the tensor-core kernels' status word (synchronises the stream)."""
    if os.environ.get("TRI_B200_CHECK") == "1" and last_path() == "tcgen05":
        check(load().tri_ws_status(ctypes.c_void_p(ws.data_ptr()), stream), "device status")


def last_path() -> str:
    return load().tri_last_path().decode()


def launch_count() -> int:
    return int(load().tri_launch_count())


def reset_launch_count() -> None:
    load().tri_reset_launch_count()


def profile_enable(on: bool) -> None:
    load().tri_profile_enable(1 if on else 0)


def profile_summary() -> dict:
    """{kernel name: (launches, total_ms, flops, bytes)} recorded since profile_enable(True)."""
    buf = ctypes.create_string_buffer(1 << 16)
    check(load().tri_profile_summary(buf, len(buf)), "tri_profile_summary")
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms, flops, nbytes = line.rsplit(" ", 4)
        out[name] = (int(n), float(ms), float(flops), float(nbytes))
    return out


def abi_field(name: str) -> str:
    return _ABI_FIELD[name]
