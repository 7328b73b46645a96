"""ctypes bindings of include/xdlb200.h (libxdlb200.so)."""
import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libxdlb200.so")

XB_F32, XB_I32, XB_I64, XB_F16, XB_BF16 = 1, 2, 10, 12, 14
XB_REC64 = 110
XB_UDF_SUM, XB_UDF_AVG, XB_UDF_ASSIGN = 0, 1, 2
XB_TRUNC_ORDER, XB_TRUNC_REVERSE = 0, 1
XB_EPI_NONE, XB_EPI_PRELU, XB_EPI_DICE, XB_EPI_SIGMOID = 0, 1, 2, 3
XB_BIAS_NONE, XB_BIAS_ROW, XB_BIAS_FULL = 0, 1, 2
XB_ATT_ENGINE_PAIR, XB_ATT_ENGINE_SPLIT = 3, 4
XB_GEMM_AUTO, XB_GEMM_SIMT, XB_GEMM_TCGEN05 = 0, 1, 2
XB_ACT_NONE, XB_ACT_SIGMOID, XB_ACT_DICE = 0, 1, 2
XB_MAX_POOL_ITEMS, XB_MAX_POOL_GROUPS = 4, 32
(XB_EW_ADD, XB_EW_SUB, XB_EW_MUL, XB_EW_DIV, XB_EW_MAX, XB_EW_MIN, XB_EW_EQ, XB_EW_NE,
 XB_EW_BROADCAST_TO, XB_EW_WHERE) = range(10)

vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class TableDesc(C.Structure):
    _fields_ = [("weights", vp), ("rows", i64), ("dim", i32), ("dtype", i32), ("row_pitch_bytes", i64),
                ("slot_keys", vp), ("slot_rows", vp), ("slots", i64)]


class PoolItem(C.Structure):
    _fields_ = [("udf", i32), ("trunc_dir", i32), ("trunc_num", i32), ("assign_stride", i32), ("out", vp),
                ("stride", i64)]


class PoolGroup(C.Structure):
    _fields_ = [("table", C.POINTER(TableDesc)), ("ids", vp), ("values", vp), ("segments", vp), ("n_ids", i64),
                ("batch", i64), ("dim", i32), ("id_dtype", i32), ("segments_are_offsets", i32), ("out_dtype", i32),
                ("n_items", i32), ("values_dtype", i32), ("items", PoolItem * XB_MAX_POOL_ITEMS)]


class ShardConfig(C.Structure):
    _fields_ = [("rank", i32), ("world", i32), ("dim", i32), ("n_tables", i32), ("tables", vp), ("table_segments", vp),
                ("max_ids", i64), ("partial_dtype", i32), ("capacity_factor", f32)]


class GemmArgs(C.Structure):
    _fields_ = [("M", i32), ("N", i32), ("K", i32), ("trans_a", i32), ("trans_b", i32), ("alpha", f32),
                ("beta", f32), ("A", vp), ("lda", i64), ("stride_a", i64), ("B", vp), ("ldb", i64),
                ("stride_b", i64), ("bias", vp), ("ldbias", i64), ("stride_bias", i64), ("bias_kind", i32),
                ("Y", vp), ("ldy", i64), ("stride_y", i64), ("batch", i32), ("ab_dtype", i32),
                ("bias_dtype", i32), ("y_dtype", i32), ("epilogue", i32), ("ep_a", vp), ("ep_b", vp),
                ("ep_c", vp), ("ep_count", i32), ("dice_nosqrt", i32), ("stride_ep", i64), ("engine", i32),
                ("bias_row_group", i64)]


class DinAttWeights(C.Structure):
    _fields_ = [("W0", vp), ("W1", vp), ("W2", vp), ("b0", vp), ("b1", vp), ("b2", f32), ("gamma0", vp),
                ("mean0", vp), ("var0", vp), ("gamma1", vp), ("mean1", vp), ("var1", vp), ("packed", vp)]


class DinAttArgs(C.Structure):
    _fields_ = [("q", vp), ("ldq", i64), ("k", vp), ("ldk", i64), ("seq_len", vp), ("out", vp), ("ldo", i64),
                ("scores", vp), ("requests", i32), ("n_cand", i32), ("T", i32), ("d", i32), ("h0", i32),
                ("h1", i32), ("act", i32), ("use_softmax", i32), ("engine", i32), ("w", DinAttWeights)]


class DinTowerArgs(C.Structure):
    _fields_ = [("user", vp), ("ldu", i64), ("q", vp), ("ldq", i64), ("k", vp), ("ldk", i64), ("att", vp), ("ldatt", i64),
                ("prob", vp), ("requests", i32), ("n_cand", i32), ("T", i32), ("d", i32), ("du", i32), ("n1", i32),
                ("n2", i32), ("n3", i32), ("W1", vp), ("b1", vp), ("gamma1", vp), ("mean1", vp), ("var1", vp),
                ("W2", vp), ("b2", vp), ("gamma2", vp), ("mean2", vp), ("var2", vp), ("W3", vp), ("b3", vp),
                ("softmax", i32), ("packed", vp)]


# every symbol include/xdlb200.h declares: (restype, argtypes)
SYMBOLS = {
    "xb_last_error": (C.c_char_p, []),
    "xb_version": (C.c_char_p, []),
    "xb_device_status": (i32, [C.POINTER(i32)]),
    "xb_device_status_clear": (i32, []),
    "xb_device_status_mirror": (i32, [C.POINTER(C.POINTER(i32))]),
    "xb_selftest_wait_timeout": (i32, [i64, vp]),
    "xb_table_row_pitch": (i64, [i32, i32]),
    "xb_table_create": (i32, [C.POINTER(C.POINTER(TableDesc)), i64, i32, i32, vp, vp]),
    "xb_table_clone": (i32, [C.POINTER(C.POINTER(TableDesc)), C.POINTER(TableDesc), i32]),
    "xb_table_destroy": (None, [C.POINTER(TableDesc)]),
    "xb_table_build_index_host": (i32, [vp, i64, i64, vp, vp]),
    "xb_copy_segments": (i32, [vp, i32, i64, vp]),
    "xb_embedding_pool_scratch_bytes": (C.c_size_t, [C.POINTER(PoolGroup), i32]),
    "xb_embedding_pool": (i32, [C.POINTER(PoolGroup), i32, vp, C.c_size_t, vp]),
    "xb_embedding_pool_static_max_bytes": (C.c_size_t, []),
    "xb_embedding_pool_static": (i32, [C.POINTER(PoolGroup), i32, vp]),
    "xb_route_scratch_bytes": (C.c_size_t, [i64, i32]),
    "xb_route_ids": (i32, [vp, vp, vp, i64, i64, i32, vp, vp, vp, vp, vp, C.c_size_t, vp]),
    "xb_unpack_routed": (i32, [vp, i64, vp, vp, vp]),
    "xb_tag_counts": (i32, [vp, i64, vp, i64, vp]),
    "xb_tag_counts_sources": (i32, [vp, vp, i32, vp, i64, vp]),
    "xb_shard_pool": (i32, [vp, vp, i32, vp, i32, i64, vp, vp, i32, i32, vp, i32, vp]),
    "xb_shard_combine": (i32, [vp, i32, i32, i64, i32, vp, i32, vp, i64, i64, i32, vp]),
    "xb_route_ids_padded": (i32, [vp, vp, i64, i64, i32, i64, vp, vp, vp, C.c_size_t, vp]),
    "xb_unpack_routed_padded": (i32, [vp, i32, i64, vp, vp, vp]),
    "xb_scan_counts_scratch_bytes": (C.c_size_t, [i32, i64]),
    "xb_scan_counts": (i32, [vp, i64, vp, i64, i32, i64, vp, C.c_size_t, vp]),
    "xb_shard_pool_padded": (i32, [vp, vp, i32, vp, i64, vp, i32, i64, i32, vp, i32, vp]),
    "xb_shard_unique_id": (i32, [vp]),
    "xb_shard_bucket_capacity": (i64, [i64, i32, f32]),
    "xb_shard_ctx_create": (i32, [C.POINTER(vp), vp, C.POINTER(ShardConfig)]),
    "xb_shard_ctx_destroy": (None, [vp]),
    "xb_sharded_pool": (i32, [vp, vp, vp, i64, i64, i32, vp, i64, i32, vp]),
    "xb_a2a_route": (i32, [vp, vp, vp, i64, vp]),
    "xb_a2a_return": (i32, [vp, vp]),
    "xb_shard_ctx_status": (i32, [vp, C.POINTER(i32)]),
    "xb_shard_ctx_bucket_capacity": (i64, [vp]),
    "xb_shard_ctx_device_bytes": (C.c_size_t, [vp]),
    "xb_sharded_pool_begin": (C.c_int, [vp, vp, vp, i64, vp]),
    "xb_sharded_pool_finish": (C.c_int, [vp, i64, i32, vp, i64, i32, vp]),
    "xb_sharded_pool_pool": (C.c_int, [vp, vp]),
    "xb_sharded_pool_combine": (C.c_int, [vp, i64, i32, vp, i64, i32, vp]),
    "xb_record_counts_padded": (C.c_int, [vp, i32, i64, vp, i64, vp]),
    "xb_shard_pool_records": (C.c_int, [vp, vp, i32, vp, i64, vp, i32, i64, i32, vp, i32, vp]),
    "xb_gather_probe": (C.c_int, [C.POINTER(TableDesc), vp, i64, vp, vp]),
    "xb_shard_ctx_profile": (C.c_int, [vp, i32]),
    "xb_shard_ctx_phase_ms": (C.c_int, [vp, vp]),
    "xb_gemm": (i32, [C.POINTER(GemmArgs), vp]),
    "xb_gemm_uses_tcgen05": (i32, [C.POINTER(GemmArgs)]),
    "xb_pack_weight_kmajor": (i32, [vp, i32, i32, i32, i64, vp, i32, i64, i32, i64, i64, vp]),
    "xb_din_attention": (i32, [C.POINTER(DinAttArgs), vp]),
    "xb_din_attention_packed_bytes": (C.c_size_t, [i32, i32, i32]),
    "xb_din_attention_pack": (i32, [C.POINTER(DinAttArgs), vp, C.c_size_t, vp]),
    "xb_din_tower_packed_bytes": (C.c_size_t, [i32, i32, i32, i32]),
    "xb_din_tower_pack": (i32, [C.POINTER(DinTowerArgs), vp, C.c_size_t, vp]),
    "xb_din_tower_workspace_bytes": (C.c_size_t, [i32, i32, i32]),
    "xb_din_tower": (i32, [C.POINTER(DinTowerArgs), vp, C.c_size_t, vp]),
    "xb_din_tower_input": (i32, [vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, i32, i32, i32, i32, i32, vp]),
    "xb_din_tower_input_split": (i32, [vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, i32, i32, i32, i32, i32, vp]),
    "xb_gru": (i32, [vp, vp, i64, i32, i32, vp, vp, vp, vp, i32, vp]),
    "xb_augru": (i32, [vp, vp, vp, i64, i32, i32, vp, vp, vp, vp, i32, vp]),
    "xb_augru_shared": (i32, [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, i32, vp]),
    "xb_dice": (i32, [vp, vp, i64, i32, vp, vp, vp, i32, i32, vp]),
    "xb_prelu": (i32, [vp, vp, i64, vp, i64, i32, i32, vp]),
    "xb_sigmoid": (i32, [vp, vp, i64, i32, vp]),
    "xb_softmax": (i32, [vp, vp, i64, i32, i64, i32, vp]),
    "xb_batchnorm": (i32, [vp, vp, i64, i32, vp, vp, vp, vp, f32, i32, i32, vp]),
    "xb_elementwise": (i32, [i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp]),
    "xb_copy2d": (i32, [vp, i64, i32, vp, i64, i32, i64, i64, vp]),
    "xb_reduce_sum": (i32, [vp, vp, i64, i64, i64, i32, vp]),
}


def build_native(verbose=False):
    """Compile csrc/ for sm_100a (nvcc cross-compiles without a GPU)."""
    cmd = ["make", "-s", "-j8", "-C", os.path.join(HERE, "csrc")]
    subprocess.check_call(cmd, stdout=None if verbose else subprocess.DEVNULL)
    host = os.path.join(HERE, "host", "Makefile")
    if os.path.exists(host):
        subprocess.check_call(["make", "-s", "-j8", "-C", os.path.join(HERE, "host")],
                              stdout=None if verbose else subprocess.DEVNULL)


_lib = None


def lib():
    """The kernel library. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


class XbError(RuntimeError):
    pass


def check(rc):
    if rc != 0:
        raise XbError("xb error %d: %s" % (rc, lib().xb_last_error().decode()))
