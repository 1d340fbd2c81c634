"""ctypes binding of libq4cuda.so: one Python attribute per symbol declared in
include/q4cuda.h, with the argument types spelled out.

The library is the product; this module only loads it.  There is no fallback:
if the shared object is missing, `load()` raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libq4cuda.so")

vp = C.c_void_p
u8p = C.c_void_p
u32 = C.c_uint32
u64 = C.c_uint64
i32 = C.c_int32
f32 = C.c_float
b = C.c_bool
sz = C.c_size_t

# name -> (restype, [argtypes]); kept in the order of include/q4cuda.h
SIGNATURES = {
    "q4_hip_init": (b, []),
    "q4_hip_shutdown": (None, []),
    "q4_hip_ok": (b, []),
    "q4_hip_stream": (vp, []),
    "q4_hip_sync": (None, []),
    "q4_hip_stream_sync": (b, []),
    "q4_hip_malloc": (vp, [sz]),
    "q4_hip_free": (None, [vp]),
    "q4_hip_h2d": (b, [vp, vp, sz]),
    "q4_hip_d2h": (b, [vp, vp, sz]),
    "q4_hip_h2d_async": (b, [vp, vp, u64]),
    "q4_hip_d2h_async": (b, [vp, vp, u64]),
    "q4_hip_fill": (b, [vp, f32, u64]),
    "q4_hip_copy_async": (b, [vp, vp, u64]),
    "q4_hip_vram_free": (u64, []),
    "q4_hip_host_alloc_coh": (vp, [sz]),
    "q4_hip_host_free_coh": (None, [vp]),
    "q4_hip_experts_alloc_a": (b, [C.c_int, u32, u64]),
    "q4_hip_experts_free_a": (None, [C.c_int]),
    "q4_hip_experts_n_a": (u32, [C.c_int]),
    "q4_hip_experts_put_a": (b, [C.c_int, u32, vp, u64]),
    "q4_hip_experts_put_async_a": (b, [C.c_int, u32, vp, u64]),
    "q4_hip_experts_dev_a": (vp, [C.c_int, u32]),
    "q4_hip_experts_base_a": (vp, [C.c_int]),
    "q4_hip_experts_stride_a": (u64, [C.c_int]),
    "q4_hip_experts_alloc": (b, [u32, u64]),
    "q4_hip_experts_free": (None, []),
    "q4_hip_experts_n": (u32, []),
    "q4_hip_experts_put": (b, [u32, vp, u64]),
    "q4_hip_experts_put_async": (b, [u32, vp, u64]),
    "q4_hip_experts_dev": (vp, [u32]),
    "q4_hip_copy_wait": (None, []),
    "q4_hip_graph_begin": (C.c_int, []),
    "q4_hip_graph_end": (vp, []),
    "q4_hip_graph_nodes": (u32, [vp]),
    "q4_hip_graph_launch": (b, [vp]),
    "q4_hip_graph_free": (None, [vp]),
    "q4_hip_moe_tok_ok": (b, [u32, u32, u32, u32, u32]),
    "q4_hip_moe_exec": (b, [vp, u64, vp, vp, u32, u32, u64, u32, u64, u32, u64, vp, vp, vp, vp,
                            vp, u32, u32, u32]),
    "q4_hip_moe_exec_dev": (b, [vp, u64, vp, vp, vp, u32, u64, u32, u64, u32, u64, vp, vp, vp,
                                vp, vp, u32, u32, u32]),
    "q4_hip_moe_stage": (b, [vp, vp, u32]),
    "q4_hip_moe_exec_staged": (b, [vp, u64, u32, u64, u32, u64, u32, u64, vp, vp, vp, vp, vp,
                                   u32, u32, u32]),
    "q4_hip_moe_scratch_warm": (None, []),
    "q4_hip_softmax_topk": (b, [vp, u32, u32, vp, vp]),
    "q4_hip_softmax_topk_launch": (b, [vp, u32, u32, vp, vp]),
    "q4_hip_grouped_rms": (b, [vp, vp, vp, u32, u32, f32]),
    "q4_hip_grouped_rms_n": (b, [vp, vp, vp, u32, u32, f32, u32]),
    "q4_hip_hc_combine": (b, [vp, vp, vp, u32, u32]),
    "q4_hip_hc_combine_n": (b, [vp, vp, vp, u32, u32, u32]),
    "q4_hip_hc_comb_rms": (b, [vp, vp, vp, vp, vp, u32, u32, f32]),
    "q4_hip_hc_comb_rms_n": (b, [vp, vp, vp, vp, vp, vp, u32, u32, f32, u32]),
    "q4_hip_gemv_dd": (b, [u32, vp, u64, u64, vp, vp, f32]),
    "q4_hip_gemv_dd_n": (b, [u32, vp, u64, u64, vp, vp, f32, u32]),
    "q4_mmq_on": (C.c_int, []),
    "q4_mmq_group": (u32, []),
    "q4_mmq_supported": (b, [u32, u64]),
    "q4_mmq_q8_bytes": (u64, [u64, u64]),
    "q4_mmq_pad": (u64, [u64]),
    "q4_mmq_quantize": (b, [vp, vp, vp, u32, u64, u64]),
    "q4_mmq_mul_id": (b, [vp, u32, u64, u64, u64, u32, vp, vp, u32, u64, vp, u64]),
    "q4_mmq_swiglu": (b, [vp, vp, u64, u64]),
    "q4_hip_expert_reduce": (b, [vp, vp, vp, vp, u32, u32, u32]),
    "q4_hip_route_pf": (b, [vp, vp, vp, u32, u32, u32]),
    "q4_hip_assign_pf": (b, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32]),
    "q4_hip_moe_win_ok": (b, [u32, u32, u32, u32, u32, u32]),
    "q4_hip_moe_exec_win": (b, [vp, u64, vp, vp, vp, u32, u32, u64, u32, u64, u32, u64, vp, vp, vp,
                                u32, u32, u32]),
    "q4_hip_clear": (None, []),
    "q4_hip_silu": (b, [vp, u64]),
    "q4_hip_sigmoid": (b, [vp, u64]),
    "q4_hip_scale": (b, [vp, f32, u64]),
    "q4_hip_scale_silu": (b, [vp, f32, u64]),
    "q4_hip_mul": (b, [vp, vp, vp, u64]),
    "q4_hip_add": (b, [vp, vp, vp, u64]),
    "q4_hip_mul_sig": (b, [vp, vp, vp, u64]),
    "q4_hip_silu_mul": (b, [vp, vp, u64]),
    "q4_hip_axpy": (b, [vp, vp, f32, u64]),
    "q4_hip_axpy_dalpha": (b, [vp, vp, vp, u64]),
    "q4_hip_axpy_rows": (b, [vp, vp, vp, u32, u32]),
    "q4_hip_dot": (b, [vp, vp, vp, u32]),
    "q4_hip_dot_sigmoid": (b, [vp, vp, vp, u32]),
    "q4_hip_sgate_axpy": (b, [vp, vp, vp, vp, u32, u32]),
    "q4_hip_moe_pack": (b, [vp, vp, vp, vp, vp, u32, b, vp, vp, u32]),
    "q4_hip_moe_final": (b, [vp, vp, vp, vp, vp, vp, u32, u32]),
    "q4_hip_gemv_m": (b, [vp, u32, vp, u32]),
    "q4_hip_moe_exec_tok": (b, [vp, u64, vp, vp, vp, u32, u32, u64, u32, u64, u32, u64, vp, vp, vp, vp,
                                u32, u32, u32]),
    "q4_mmvq_n": (b, [u32, vp, u64, u64, vp, vp, f32, u32]),
    "q4_mmvq_warm": (None, []),
    "q4_mmvq_hold": (None, [vp]),
    "q4_mmvq_release": (None, []),
    "q4_mmvq_on": (C.c_int, []),
    "q4_mmvq_verify": (None, [C.c_int]),
    "q4_mmvq_set": (None, [C.c_int]),
    "q4_mmq_wbuf": (b, [u64, u64, u32, vp, vp]),
    "q4_mmq_wbuf_lend": (b, [vp, u64, vp, u64]),
    "q4_mmq_gather": (b, [vp, u64, u64, u64, u64, u64, u64, u64, vp, vp, u32, vp, vp]),
    "q4_xg_on": (C.c_int, []),
    "q4_hip_host_register": (b, [vp, sz]),
    "q4_hip_host_devptr": (vp, [vp]),
    "q4_hip_host_unregister": (None, [vp]),
    "q4_hip_copy_memset": (b, [vp, C.c_int, sz]),
    "q4_hip_gemv": (b, [u32, vp, u64, u64, vp, vp, f32]),
    "q4_hip_gemv_dev": (b, [u32, vp, u64, u64, vp, vp, f32]),
    "q4_hip_gemv_dd_n_which": (b, [u32, vp, u64, u64, vp, vp, f32, u32, vp]),
    "q4_hip_moe_act": (b, [vp, vp, u64]),
    "q4_hip_mark_pt": (None, [C.c_int]),
    "q4_hip_moe_pf": (b, [u32, vp, u64, u64, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "q4_hip_moe_pf2": (b, [u32, vp, u64, u64, u64, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "q4_hip_moe_wmma": (b, [u32, vp, u64, u64, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "q4_hip_moe_wmma2": (b, [u32, vp, u64, u64, u64, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "q4_hip_gateup_q4k": (b, [vp, vp, vp, vp, u32, u32]),
    "q4_hip_gateup_q4k_n_which": (b, [vp, vp, vp, vp, u32, u32, u32, vp]),
    "q4_hip_q8_reuse": (b, [vp, u64, u64, vp, vp, vp, f32, u32]),
    "q4_xg_gu_type": (b, [u32]),
    "q4_xg_dn_type": (b, [u32]),
    "q4_xg_shape_ok": (b, [u32, u32]),
    "q4_xg_tile_cap": (u32, [u32, u32]),
    "q4_xg_tiles": (u32, [vp, vp, vp, u32, vp, u32]),
    "q4_xg_cvt": (b, [vp, vp, u64]),
    "q4_xg_gu": (b, [u32, vp, u64, u64, u64, u32, u32, vp, u32, vp, vp, vp]),
    "q4_xg_dn": (b, [u32, vp, u64, u64, u32, u32, vp, u32, vp, vp]),
    "q4_hip_route_dev": (b, [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, vp, vp, vp, vp, u32, u32]),
    "q4_hip_route_dev_n": (b, [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32]),
    "q4_hip_cpx_wait": (b, [vp, vp, vp]),
    "q4_hip_cpx_spin_init": (b, []),
    "q4_hip_cpx_spin": (b, [vp, vp]),
    "q4_hip_cpx_wait_timeouts": (C.c_ulonglong, []),
    "q4_hip_cpx_wait_reset": (None, []),
    "q4_hip_cpx_wait_lastseen": (C.c_ulonglong, []),
    "q4_hip_pred_size": (sz, []),
    "q4_hip_pred_sel": (b, [vp, vp, vp, vp, vp, u32, u32, u32, f32]),
    "q4_hip_vtl_init": (b, []),
    "q4_hip_vtl_stamp": (b, [u32]),
    "q4_hip_vtl_read": (b, [vp, u32, C.c_double]),
    "q4_hip_vtl_calib": (C.c_double, []),
    "q4_cuda_quant8": (b, [vp, u64, vp, vp, vp]),
    "q4_cuda_fmt_dequant": (b, [u32, vp, u64, u64, vp]),
    "q4_cuda_fmt_idot": (b, [u32, vp, u64, u64, vp, vp]),
    "q4_cuda_iq4nl_dequant": (b, [vp, u64, u64, vp]),
    "q4_cuda_iq4nl_idot": (b, [vp, u64, u64, vp, vp]),
    "q4_cuda_iq4_dequant": (b, [u32, vp, u64, u64, vp]),
    "q4_cuda_iq4_idot": (b, [u32, vp, u64, u64, vp, vp]),
    "q4_cuda_iq3s_dequant": (b, [vp, u64, u64, vp]),
    "q4_cuda_iq3s_idot": (b, [vp, u64, u64, vp, vp]),
    "q4_cuda_moe_decode": (b, [vp, u64, u64, u64, u64, i32, vp, vp, f32, vp, u32, u32, u32, u32,
                               vp, vp, vp]),
    "q4_cuda_moe_layer_n_ws_bytes": (u64, [u32, u32, u32, u32, u32]),
    "q4_cuda_moe_layer_n": (b, [vp, u64, u64, u64, u64, i32, vp, vp, f32, vp, u32, u32, u32, u32,
                                u32, vp, vp, vp, vp, u64]),
    "q4_cuda_route_small": (b, [vp, vp, f32, vp, u32, u32, u32, u32, vp, vp, vp, vp]),
    "q4_cuda_moe_layer_nt": (b, [vp, u64, u32, u64, u64, u32, u64, i32, vp, vp, f32, vp, u32, u32, u32, u32,
                                 u32, vp, vp, vp, vp, u64]),
    "q4_cuda_moe_exec_noalloc": (b, [vp, u64, vp, vp, u32, u64, u64, u64, vp, vp, vp, u32, u32, u32,
                                     vp]),
    "q4_cuda_set_tiled_default": (None, [C.c_int]),
    "q4_cuda_experts_tiled_a": (C.c_int, [C.c_int]),
    "q4_cuda_experts_retile_a": (b, [C.c_int, u32, u32]),
    "q4_cuda_experts_get_a": (b, [C.c_int, u32, vp, u64]),
    "q4_cuda_moe_decode_host": (b, [vp, u64, u64, u64, u64, i32, vp, vp, f32, vp, u32, u32, u32,
                                    u32, vp]),
    "q4_cuda_decode_plan": (vp, [vp, u64, u64, u64, u64, i32, vp, f32, vp, u32, u32, u32, u32]),
    "q4_cuda_decode_plan_dev": (b, [vp, vp, vp, vp, vp]),
    "q4_cuda_decode_plan_host": (b, [vp, vp, vp]),
    "q4_cuda_decode_plan_free": (None, [vp]),
    "q4_cuda_decode_stack_plan": (vp, [vp, u32, u64, u64, u64, u64, i32, f32, u32, u32, u32, u32]),
    "q4_cuda_decode_stack_layers": (u32, [vp]),
    "q4_cuda_decode_stack_dev": (b, [vp, vp, vp, vp, vp]),
    "q4_cuda_decode_stack_host": (b, [vp, vp, vp]),
    "q4_cuda_decode_stack_free": (None, [vp]),
    "q4_cuda_decode_stack_set_sgate": (b, [vp, u32, vp]),
    "q4_cuda_decode_stack_set_final": (b, [vp, vp, vp, u32]),
    "q4_cuda_decode_session_begin": (vp, [vp, u32, u32, u32]),
    "q4_cuda_decode_session_step": (b, [vp, vp, vp]),
    "q4_cuda_decode_session_end": (b, [vp]),
    "q4_cuda_fused_profile_enable": (b, [C.c_int]),
    "q4_cuda_fused_profile_layer": (None, [u32]),
    "q4_cuda_decode_wait_limit": (None, [u32]),
    "q4_cuda_fused_profile_read": (u32, [vp, u32]),
    "q4_cuda_mmq_swiglu_quantize": (b, [vp, vp, u64, u64]),
    "q4_cuda_expert_reduce_set": (b, [vp, vp, vp, vp, u32, u32, u32]),
    "q4_cuda_assign_local": (b, [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, C.c_int, u32, u32]),
    "q4_cuda_mmq_tc_mode": (b, [C.c_int]),
    "q4_cuda_mmq_q8_compat": (None, [C.c_int]),
    "q4_cuda_mmq_q8_sections": (b, [vp, u64, u64, vp, vp, vp]),
    "q4_cuda_synth_iq3s": (b, [vp, u64, u64]),
    "q4_cuda_synth_iq3s_at": (b, [vp, u64, u64, u64]),
    "q4_cuda_synth_normal": (b, [vp, u64, u64, f32, f32]),
    "q4_cuda_timer_begin": (b, []),
    "q4_cuda_timer_end": (b, []),
    "q4_cuda_timer_ms": (f32, []),
    "q4_cuda_timer_mark": (b, [u32]),
    "q4_cuda_timer_between_ms": (f32, [u32, u32]),
    "q4_cuda_launch_count": (u64, []),
    "q4_cuda_device_error": (u32, []),
}

_lib = None


def load():
    """dlopen the library and attach signatures.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libq4cuda.so is not built (run `python suzuku-engine-q4_b200/build.py`); "
            "this package has no other compute path")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


EP_LIB_PATH = os.path.join(_HERE, "libq4cuda_ep.so")
EP_SIGNATURES = {
    "q4_cuda_ep_unique_id": (b, [vp]),
    "q4_cuda_ep_init": (b, [vp, C.c_int, C.c_int]),
    "q4_cuda_ep_shutdown": (None, []),
    "q4_cuda_ep_rank": (C.c_int, []),
    "q4_cuda_ep_world": (C.c_int, []),
    "q4_cuda_ep_allreduce_max": (b, [vp]),
    "q4_cuda_ep_allreduce_mode": (C.c_int, [C.c_int]),
    "q4_cuda_ep_split_routing": (None, [C.c_int]),
    "q4_cuda_ep_error": (u32, []),
    "q4_cuda_ep_layer_ws_bytes": (u64, [u32, u32, u32, u32, u32, u32]),
    "q4_cuda_ep_layer": (b, [vp, u64, u64, u64, u64, C.c_int, vp, vp, f32, vp, u32, u32, u32, u32, u32,
                             vp, vp, u64]),
    "q4_cuda_ep_layer_ar": (b, [vp, u64, u64, u64, u64, C.c_int, vp, vp, f32, vp, u32, u32, u32, u32, u32,
                                vp, vp, u64]),
    "q4_cuda_ep_exchange_floor_us": (b, [u32, u32, u32, u32, u32, vp, u64, u32, vp]),
}
_ep = None


def load_ep():
    """The expert-parallel library (links NCCL); load() must have succeeded first."""
    global _ep
    if _ep is not None:
        return _ep
    load()
    if not os.path.exists(EP_LIB_PATH):
        raise RuntimeError("libq4cuda_ep.so is not built (run `python suzuku-engine-q4_b200/build.py`)")
    lib = C.CDLL(EP_LIB_PATH)
    for name, (res, args) in EP_SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _ep = lib
    return lib
