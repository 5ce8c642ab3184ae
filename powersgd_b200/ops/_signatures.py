"""ctypes prototypes of the exported C entry points."""
import ctypes as C

vp = C.c_void_p
i32 = C.c_int
f32 = C.c_float


def declare(lib) -> None:
    lib.psgd_last_error.restype = C.c_char_p
    lib.psgd_last_error.argtypes = []
    lib.psgd_version.restype = i32
    lib.psgd_device_info.restype = i32
    lib.psgd_device_info.argtypes = [C.POINTER(i32)] * 4

    lib.psgd_orth_launch.restype = i32
    lib.psgd_orth_launch.argtypes = [vp, i32, vp, i32, i32, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp]

    lib.psgd_gemm_nn_tile_rows.restype = i32
    lib.psgd_gemm_nn_tile_rows.argtypes = [i32]
    lib.psgd_gemm_nt_max_rows.restype = i32
    lib.psgd_gemm_nt_max_rows.argtypes = [i32]
    lib.psgd_gemm_template_rank.restype = i32
    lib.psgd_gemm_template_rank.argtypes = [i32]
    lib.psgd_gemm_ffma_launch.restype = i32
    lib.psgd_gemm_ffma_launch.argtypes = [i32, i32, vp, vp, i32, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp]

    lib.psgd_finalize_launch.restype = i32
    lib.psgd_finalize_launch.argtypes = [vp, vp, i32, i32, i32, vp, i32, vp, vp, vp, vp, f32, i32, vp, i32, vp, vp, i32, f32, vp]
    lib.psgd_finalize_uses_strip.restype = i32
    lib.psgd_finalize_uses_strip.argtypes = [i32, i32, i32, i32]

    lib.psgd_flat_block_elems.restype = i32
    lib.psgd_flat_block_elems.argtypes = []
    lib.psgd_flat_launch.restype = i32
    lib.psgd_flat_launch.argtypes = [i32, i32, vp, vp, vp, i32, vp, vp, f32, vp, C.c_longlong, i32, vp]

    for name, sig in _OPTIONAL.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.restype, fn.argtypes = sig


# entry points that later translation units add; declared when present
i64 = C.c_longlong
_OPTIONAL = {
    "psgd_sign_pack": (i32, [vp, i64, vp, vp]),
    "psgd_sign_unpack": (i32, [vp, i64, f32, vp, i32, vp]),
    "psgd_sign_vote": (i32, [vp, i32, i64, i32, vp, vp, vp]),
    "psgd_gemm_tc_rank_pad": (i32, [i32]),
    "psgd_tma_encode_matrix": (i32, [vp, vp, i32, i32]),
    "psgd_gemm_tc_launch": (i32, [i32, i32, i32, vp, vp, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp]),
    "psgd_finalize_strip_rows": (i32, [i32, i32]),
    "psgd_orth_template_rank": (i32, [i32]),
    "psgd_orth_chunk_rows": (i32, [i32]),
    "psgd_orth_part_doubles": (i32, [i32, i32]),
    "psgd_finalize_tc_max_k": (i32, []),
    "psgd_finalize_tc_launch": (i32, [vp, vp, i32, vp, vp, i32, i32, vp, vp, vp, vp, f32, i32, vp, vp]),
    "psgd_topk_workspace_ints": (i32, []),
    "psgd_topk_abs": (i32, [vp, i64, i64, vp, vp, vp, vp, vp]),
    "psgd_topk_item_bytes": (i32, []),
    "psgd_topk_abs_many": (i32, [vp, i32, vp, vp, vp, i32, vp, vp, vp, vp]),
    "psgd_sparse_combine_max_segments": (i32, []),
    "psgd_sparse_combine_launch": (i32, [vp, vp, i32, i64, vp, i32, f32, vp, vp, vp]),
    "psgd_svd_tall_max_cols": (i32, []),
    "psgd_svd_tall_launch": (i32, [vp, i32, vp, vp, vp, vp, vp]),
    "psgd_bulk_chunk_floats": (i64, []),
    "psgd_bulk_arena_bytes": (i64, [i64, i32]),
    "psgd_bulk_allreduce_launch": (i32, [vp, i64, i32, vp]),
    "psgd_bulk_finish_launch": (i32, [vp, i64, i32, vp]),
    "psgd_mc_buffer_bytes": (i32, []),
    "psgd_mc_supported": (i32, []),
    "psgd_mc_round_up": (i32, [i32, C.c_ulonglong, vp]),
    "psgd_mc_create": (i32, [i32, C.c_ulonglong, vp, vp]),
    "psgd_mc_import": (i32, [i32, C.c_ulonglong, vp]),
    "psgd_mc_add_device": (i32, [vp]),
    "psgd_mc_bind": (i32, [vp]),
    "psgd_mc_release": (i32, [vp]),
    "psgd_nvls_allreduce_fused_launch": (i32, [vp, vp, i64, i32, i32, vp]),
    "psgd_nvls_allreduce_launch": (i32, [vp, i64, i32, i32, i32, vp]),
    "psgd_read_pass_launch": (i32, [vp, i64, vp, i32, vp]),
    "psgd_finalize_uses_strip": (i32, [i32, i32, i32, i32]),
    "psgd_symm_alloc": (i32, [C.c_size_t, C.POINTER(vp)]),
    "psgd_symm_free": (i32, [vp]),
    "psgd_symm_handle_bytes": (i32, []),
    "psgd_symm_export": (i32, [vp, vp]),
    "psgd_symm_import": (i32, [vp, C.POINTER(vp)]),
    "psgd_symm_unmap": (i32, [vp]),
    "psgd_status_alloc": (i32, [C.POINTER(C.POINTER(i32)), C.POINTER(C.POINTER(i32))]),
    "psgd_status_free": (i32, [C.POINTER(i32)]),
    "psgd_comm_desc_bytes": (i32, []),
    "psgd_comm_fill": (i32, [vp, i32, i32, vp, vp, vp, i64, C.c_double]),
    "psgd_factor_reduce_launch": (i32, [vp, i64, vp, vp, vp]),
    "psgd_allreduce_oneshot_launch": (i32, [vp, vp, vp, i64, f32, i32, vp]),
    "psgd_allgather_oneshot_launch": (i32, [vp, vp, vp, i64, i32, vp]),
}
