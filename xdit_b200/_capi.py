"""ctypes binding of ``libxdit_b200.so`` (declarations mirror ``include/xdit_b200.h``).

The library is the product: there is no Python or CPU fallback behind it.  ``load()`` raises
``RuntimeError`` when the shared object is missing, and every compute wrapper in
``xdit_b200.ops`` raises when it is handed a tensor that is not on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# XDIT_B200_LIB selects another build of the same library (same ABI), e.g. one compiled with other options
LIB_PATH = os.environ.get("XDIT_B200_LIB") or os.path.join(_PKG, "libxdit_b200.so")

XDIT_BF16, XDIT_F16, XDIT_F32 = 0, 1, 2
XDIT_MAX_PACK_JOBS = 4
XDIT_MAX_OUT_SEGMENTS = 16
XDIT_PEER_HANDLE_BYTES = 64
XDIT_STATIC_ACC_FLOATS = 8 * 1024 * 1024

EXPORTS = [
    "xdit_query_caps",
    "xdit_last_error_string",
    "xdit_attn_fwd",
    "xdit_attn_split_scratch_bytes",
    "xdit_attn_which",
    "xdit_attn_fwd_static_acc",
    "xdit_ulysses_pack",
    "xdit_ulysses_pack_peers",
    "xdit_peer_alloc",
    "xdit_peer_open",
    "xdit_peer_close",
    "xdit_peer_free",
    "xdit_peer_barrier",
    "xdit_peer_copy",
    "xdit_ulysses_pack_out",
    "xdit_ulysses_unpack_out",
    "xdit_ulysses_unpack_in",
    "xdit_kv_patch_update",
    "xdit_seq_shard_pad",
    "xdit_seq_gather_unpad",
    "xdit_merge_out_lse",
    "xdit_qk_norm_rope_pack",
]


ABI_VERSION = 3  # XDIT_ABI_VERSION of include/xdit_b200.h: the structures below mirror that header


class Caps(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int), ("device", C.c_int), ("sm_major", C.c_int), ("sm_minor", C.c_int),
        ("sm_count", C.c_int), ("max_smem_per_block", C.c_int), ("supported", C.c_int),
    ]


class Seq(C.Structure):
    _fields_ = [
        ("ptr", C.c_void_p),
        ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_seg", C.c_int64), ("stride_row", C.c_int64),
        ("nseg", C.c_int32), ("seg_len", C.c_int32),
    ]


class AttnParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("H", C.c_int32), ("D", C.c_int32),
        ("q", Seq), ("k", Seq), ("v", Seq), ("k2", Seq), ("v2", Seq),
        ("out", C.c_void_p),
        ("out_stride_b", C.c_int64), ("out_stride_h", C.c_int64), ("out_stride_seg", C.c_int64),
        ("out_stride_row", C.c_int64),
        ("lse", C.c_void_p), ("o_acc", C.c_void_p), ("lse_acc", C.c_void_p),
        ("acc_in", C.c_int32), ("acc_out", C.c_int32), ("causal", C.c_int32),
        ("softmax_scale", C.c_float), ("force_generic", C.c_int32),
        ("status", C.c_void_p),
        ("status_host", C.c_void_p), ("wait_limit_ns", C.c_uint32), ("selftest_stall", C.c_int32),
        ("out_segments", C.POINTER(C.c_void_p)),
        ("split_scratch", C.c_void_p),
        ("split_scratch_bytes", C.c_int64),
    ]


class PackJob(C.Structure):
    _fields_ = [
        ("src", C.c_void_p),
        ("src_stride_b", C.c_int64), ("src_stride_h", C.c_int64), ("src_stride_row", C.c_int64),
        ("joint", C.c_void_p),
        ("joint_stride_b", C.c_int64), ("joint_stride_h", C.c_int64), ("joint_stride_row", C.c_int64),
        ("dst", C.c_void_p), ("dst_peer_stride", C.c_int64),
        ("s", C.c_int32), ("s_joint", C.c_int32), ("joint_front", C.c_int32),
        ("src_stride_peer", C.c_int64), ("joint_stride_peer", C.c_int64),
    ]


class KvPatchParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("H", C.c_int32), ("D", C.c_int32),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("cache_stride_b", C.c_int64), ("cache_stride_h", C.c_int64), ("cache_stride_row", C.c_int64),
        ("cache_rows", C.c_int32),
        ("k_new", Seq), ("v_new", Seq),
        ("row_start", C.c_int32),
    ]


class PrologueParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32), ("B", C.c_int32), ("H", C.c_int32), ("D", C.c_int32), ("s", C.c_int32),
        ("U", C.c_int32), ("norm_per_head", C.c_int32), ("eps", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_row", C.c_int64), ("k_stride_b", C.c_int64),
        ("k_stride_row", C.c_int64), ("v_stride_b", C.c_int64), ("v_stride_row", C.c_int64),
        ("norm_q_weight", C.c_void_p), ("norm_k_weight", C.c_void_p),
        ("cos", C.c_void_p), ("sin", C.c_void_p), ("cos_sin_stride_row", C.c_int64),
        ("dst_q", C.c_void_p), ("dst_k", C.c_void_p), ("dst_v", C.c_void_p),
        ("dst_q_peer_stride", C.c_int64), ("dst_k_peer_stride", C.c_int64), ("dst_v_peer_stride", C.c_int64),
        ("dst_stride_h", C.c_int64 * 3), ("dst_stride_b", C.c_int64 * 3),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m xdit_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = C.CDLL(LIB_PATH)
    lib.xdit_query_caps.argtypes = [C.POINTER(Caps)]
    lib.xdit_query_caps.restype = C.c_int
    caps = Caps()
    lib.xdit_query_caps(C.byref(caps))  # the version is filled in before anything that needs a GPU
    if caps.abi_version != ABI_VERSION:
        raise RuntimeError(f"{LIB_PATH} has ABI version {caps.abi_version}, these bindings are written for "
                           f"{ABI_VERSION}: rebuild it with `python -m xdit_b200.build --force`")
    lib.xdit_last_error_string.argtypes = []
    lib.xdit_last_error_string.restype = C.c_char_p
    lib.xdit_attn_fwd.argtypes = [C.POINTER(AttnParams), C.c_void_p]
    lib.xdit_attn_fwd.restype = C.c_int
    lib.xdit_attn_split_scratch_bytes.argtypes = [C.POINTER(AttnParams)]
    lib.xdit_attn_split_scratch_bytes.restype = C.c_int64
    lib.xdit_attn_fwd_static_acc.argtypes = [C.POINTER(AttnParams), C.c_void_p]
    lib.xdit_attn_fwd_static_acc.restype = C.c_int
    lib.xdit_attn_which.argtypes = [C.POINTER(AttnParams)]
    lib.xdit_attn_which.restype = C.c_int
    lib.xdit_ulysses_pack.argtypes = [C.POINTER(PackJob), C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_int32, C.c_void_p]
    lib.xdit_ulysses_pack.restype = C.c_int
    lib.xdit_ulysses_pack_peers.argtypes = [C.POINTER(PackJob), C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                            C.c_int32, C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_int64),
                                            C.c_void_p]
    lib.xdit_ulysses_pack_peers.restype = C.c_int
    lib.xdit_peer_alloc.argtypes = [C.c_int64, C.POINTER(C.c_void_p), C.c_char_p]
    lib.xdit_peer_alloc.restype = C.c_int
    lib.xdit_peer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.xdit_peer_open.restype = C.c_int
    lib.xdit_peer_close.argtypes = [C.c_void_p]
    lib.xdit_peer_close.restype = C.c_int
    lib.xdit_peer_free.argtypes = [C.c_void_p]
    lib.xdit_peer_free.restype = C.c_int
    lib.xdit_peer_barrier.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_uint32,
                                      C.c_void_p, C.c_void_p, C.c_void_p]
    lib.xdit_peer_barrier.restype = C.c_int
    lib.xdit_peer_copy.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    lib.xdit_peer_copy.restype = C.c_int
    lib.xdit_ulysses_pack_out.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                          C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    lib.xdit_ulysses_pack_out.restype = C.c_int
    for name in ("xdit_ulysses_unpack_out", "xdit_ulysses_unpack_in"):
        fn = getattr(lib, name)
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                       C.c_int32, C.c_void_p]
        fn.restype = C.c_int
    lib.xdit_seq_shard_pad.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_int32,
                                       C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    lib.xdit_seq_shard_pad.restype = C.c_int
    lib.xdit_seq_gather_unpad.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                          C.c_int32, C.c_int32, C.c_void_p]
    lib.xdit_seq_gather_unpad.restype = C.c_int
    lib.xdit_kv_patch_update.argtypes = [C.POINTER(KvPatchParams), C.c_void_p]
    lib.xdit_kv_patch_update.restype = C.c_int
    lib.xdit_qk_norm_rope_pack.argtypes = [C.POINTER(PrologueParams), C.c_void_p]
    lib.xdit_qk_norm_rope_pack.restype = C.c_int
    lib.xdit_merge_out_lse.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]
    lib.xdit_merge_out_lse.restype = C.c_int
    _lib = lib
    return lib


class XditError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str):
        super().__init__(f"{where} failed with status {code}: {detail}")
        self.code = code


def check(rc: int, where: str) -> None:
    if rc != 0:
        msg = load().xdit_last_error_string()
        raise XditError(rc, where, msg.decode() if msg else "")
