"""ctypes binding of libh3_b200.so -- the same C ABI a C caller of the reference links against.

Nothing here computes: every function forwards raw device pointers (taken from torch tensors,
which only provide device memory and streams) to the library.  Loading fails loudly when the
library has not been built; there is no fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libh3_b200.so"

F32, BF16, F16, I32 = 0, 1, 2, 3
EPI_PLAIN, EPI_GATE, EPI_SWIGLU, EPI_GELU, EPI_QKV_ROPE = 0, 1, 2, 3, 4
ERR_LEN = 512

vp = C.c_void_p
sz = C.c_size_t
i32 = C.c_int
f32 = C.c_float
cs = C.c_char_p
dbl_p = C.POINTER(C.c_double)


class H3Error(RuntimeError):
    pass


class DeviceInfo(C.Structure):
    _fields_ = [("device_index", i32), ("name", C.c_char * 256), ("compute_major", i32), ("compute_minor", i32),
                ("total_memory_bytes", sz), ("free_memory_bytes", sz), ("multiprocessor_count", i32),
                ("driver_version", i32), ("runtime_version", i32)]


class DitGemmEpi(C.Structure):  # h3_cuda_dit_gemm_epi, the reference's epilogue description
    _fields_ = [("swiglu", i32), ("gate", i32), ("d_residual", vp), ("d_modulation", vp), ("d_row_map", vp),
                ("d_lora", vp), ("lora_ready", vp), ("slots", sz), ("gate_slot", sz), ("requant_mode", i32),
                ("requant_gs", i32), ("d_rq_x", vp), ("d_rq_act", vp), ("d_rq_pre", vp), ("requant_rows", sz),
                ("y_f16", i32)]


class GemmEpi(C.Structure):  # h3b_gemm_epi
    _fields_ = [("kind", i32), ("out_dtype", i32), ("d_residual", vp), ("d_modulation", vp), ("d_row_map", vp),
                ("slots", sz), ("gate_slot", sz), ("d_key", vp), ("d_value", vp), ("d_q_norm", vp), ("d_k_norm", vp),
                ("d_rope_cos", vp), ("d_rope_sin", vp), ("rope_half", sz), ("epsilon", f32), ("round_qkv", i32),
                ("scatter", vp), ("d_lora", vp), ("lora_ready", vp)]


class NormArgs(C.Structure):  # h3b_norm_args
    _fields_ = [("d_x", vp), ("d_branch", vp), ("d_norm_w", vp), ("d_modulation", vp), ("d_row_map", vp),
                ("rows", sz), ("width", sz), ("slots", sz), ("gate_slot", sz), ("shift_slot", sz),
                ("scale_slot", sz), ("epsilon", f32), ("dtype", i32), ("identity", i32), ("convrot_gs", i32),
                ("d_gated", vp), ("d_normed", vp), ("d_rot", vp), ("d_q", vp), ("d_scales", vp), ("d_fp4", vp),
                ("d_sf", vp)]


class DitConfig(C.Structure):  # h3b_dit_config
    _fields_ = [("kind", i32), ("stream_dtype", i32), ("convrot_gs", i32), ("dim", sz), ("heads", sz),
                ("head_dim", sz), ("ffn", sz), ("rope_half", sz), ("n_blocks", sz), ("mod_rows", sz), ("t_dim", sz),
                ("eps", f32)]


class UlyssesDirect(C.Structure):  # h3b_ulysses_direct
    _fields_ = [("ulysses", i32), ("rank", i32), ("seq_local", sz), ("heads", sz), ("head_dim", sz),
                ("q", vp), ("k", vp), ("v", vp), ("att", vp),
                ("peer_q", vp * 8), ("peer_k", vp * 8), ("peer_v", vp * 8), ("peer_att", vp * 8)]


class UlyssesCfg(C.Structure):  # h3_ulysses_cfg
    _fields_ = [("tp_size", i32), ("ulysses", i32), ("ring", i32), ("rank", i32), ("world_size", i32), ("comm", vp)]


_ERR = (cs, sz)

# name -> (restype, argtypes); `_ERR` marks the trailing (char *error, size_t error_size) pair
_SIGS = {
    "h3_cuda_create": (vp, (i32,) + _ERR),
    "h3_cuda_free": (None, (vp,)),
    "h3_cuda_release_heavy_workspace": (None, (vp,)),
    "h3_cuda_pregrow_dit_scratch": (i32, (vp, sz, sz, sz, sz, sz) + _ERR),
    "h3_cuda_pregrow_hadamard": (i32, (vp, i32) + _ERR),
    "h3_cuda_dit_scratch_pregrown": (i32, (vp,)),
    "h3_cuda_bind_device": (i32, (vp,) + _ERR),
    "h3_cuda_device_count": (i32, _ERR),
    "h3_cuda_probe": (i32, (i32, C.POINTER(DeviceInfo)) + _ERR),
    "h3_cuda_get_info": (i32, (vp, C.POINTER(DeviceInfo))),
    "h3_cuda_mem_info": (i32, (vp, C.POINTER(sz), C.POINTER(sz)) + _ERR),
    "h3_cuda_set_graph_capture": (None, (vp, i32)),
    "h3_cuda_graph_capture": (i32, (vp,)),
    "h3_cuda_set_quiet": (None, (vp, i32)),
    "h3_cuda_quiet": (i32, (vp,)),
    "h3_cuda_set_op_stream": (i32, (vp, vp) + _ERR),
    "h3_cuda_op_stream": (vp, (vp,)),
    "h3_cuda_stream": (vp, (vp, i32)),
    "h3_cuda_stream_count": (i32, ()),
    "h3_cuda_event_record_default": (i32, (vp, C.POINTER(vp)) + _ERR),
    "h3_cuda_event_record": (i32, (vp, vp) + _ERR),
    "h3_cuda_stream_wait_event": (i32, (vp, vp) + _ERR),
    "h3_cuda_event_destroy": (None, (vp,)),
    "h3_cuda_host_alloc": (vp, (sz, C.POINTER(i32))),
    "h3_cuda_host_free": (None, (vp, i32)),
    "h3b_cuda_check": (i32, (vp, C.POINTER(i32)) + _ERR),
    "h3b_cuda_launch_count": (C.c_ulonglong, (vp, i32)),
    "h3b_cuda_profile_begin": (None, (vp,)),
    "h3b_cuda_profile_end": (i32, (vp, dbl_p, C.POINTER(i32), i32)),
    "h3_cuda_w4a8_weight_create": (i32, (vp, vp, sz, sz, vp, vp, vp, i32, C.POINTER(vp), dbl_p, dbl_p) + _ERR),
    "h3_cuda_w4a8_weight_create_from_i8": (i32, (vp, vp, sz, sz, vp, C.POINTER(vp), dbl_p, i32) + _ERR),
    "h3_cuda_w4a8_weight_upload_i8": (i32, (vp, vp, sz, sz, vp, i32) + _ERR),
    "h3_cuda_w4a8_weight_ensure_ready": (i32, (vp,) + _ERR),
    "h3_cuda_w4a8_weight_on_device": (i32, (vp, i32) + _ERR),
    "h3_cuda_w4a8_weight_free": (None, (vp,)),
    "h3_cuda_w4a8_weight_n": (sz, (vp,)),
    "h3_cuda_w4a8_weight_k": (sz, (vp,)),
    "h3_cuda_w4a8_weight_download_int8": (i32, (vp, vp) + _ERR),
    "h3b_w4g_weight_create": (i32, (vp, vp, vp, sz, sz, i32, C.POINTER(vp)) + _ERR),
    "h3b_w4a8_weight_data": (vp, (vp,)),
    "h3b_w4a8_weight_scales": (vp, (vp,)),
    "h3b_w4a8_weight_download_scales": (i32, (vp, vp) + _ERR),
    "h3_cuda_gemm_i8_dequant_f32": (i32, (vp, vp, vp, vp, i32, vp, sz, sz, sz, vp, dbl_p, cs, sz) + _ERR),
    "h3_cuda_gemm_i8_dequant_f32_w": (i32, (vp, vp, vp, vp, i32, sz, vp, dbl_p, cs, sz) + _ERR),
    "h3_cuda_gemm_i8_dequant_f32_w_act": (i32, (vp, vp, vp, i32, sz, vp, dbl_p, dbl_p, cs, sz) + _ERR),
    "h3_cuda_gemm_i8_dequant_f32_w_act_dev": (i32, (vp, vp, vp, i32, sz, vp, dbl_p, dbl_p, cs, sz) + _ERR),
    "h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi": (i32, (vp, vp, vp, i32, sz, vp, dbl_p, dbl_p, cs, sz,
                                                        C.POINTER(DitGemmEpi)) + _ERR),
    "h3_cuda_gemm_i8_dequant_f32_dev_pre_q": (i32, (vp, vp, vp, vp, sz, vp, dbl_p, dbl_p, cs, sz,
                                                    C.POINTER(DitGemmEpi)) + _ERR),
    "h3b_gemm_i8_dequant_f32_w_act_dev_noalloc": (i32, (vp, vp, vp, i32, sz, vp) + _ERR),
    "h3b_linear_noalloc_max_codes": (sz, ()),
    "h3b_linear_noalloc_max_rows": (sz, ()),
    "h3_cuda_convrot_act_f32_dd": (i32, (vp, vp, sz, sz, i32, vp) + _ERR),
    "h3b_gemm_i8_dev": (i32, (vp, vp, vp, vp, sz, vp, C.POINTER(GemmEpi)) + _ERR),
    "h3b_quantize_act_int8_dev": (i32, (vp, vp, i32, sz, sz, vp, vp) + _ERR),
    "h3b_norm_dev": (i32, (vp, C.POINTER(NormArgs)) + _ERR),
    "h3_cuda_adaln_f32_dev": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, f32, vp, dbl_p) + _ERR),
    "h3_cuda_gate_f32_dev": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, sz, vp, dbl_p) + _ERR),
    "h3_cuda_swiglu_f32_dev": (i32, (vp, vp, sz, sz, vp, dbl_p) + _ERR),
    "h3_cuda_gate_adaln_f32_dev": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, sz, f32, vp, vp, dbl_p) + _ERR),
    "h3_cuda_rms_norm_f32_dev": (i32, (vp, vp, vp, sz, sz, f32, vp) + _ERR),
    "h3_cuda_qkv_rope_f32_dev": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f32, vp, vp, vp, dbl_p) + _ERR),
    "h3_cuda_qkv_rope_f32_dev_layout": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f32, i32, i32, vp, vp, vp,
                                              dbl_p) + _ERR),
    "h3_cuda_f32_to_f16_dev": (i32, (vp, vp, vp, sz) + _ERR),
    "h3_cuda_f16_to_f32_dev": (i32, (vp, vp, vp, sz) + _ERR),
    "h3b_qkv_rope_dev": (i32, (vp, vp, i32, vp, vp, vp, vp, sz, sz, sz, sz, f32, i32, i32, vp, vp, vp, i32) + _ERR),
    "h3b_cast_dev": (i32, (vp, vp, i32, vp, i32, sz) + _ERR),
    "h3b_gelu_tanh_dev": (i32, (vp, vp, vp, i32, sz) + _ERR),
    "h3_cuda_sdpa_f32_dev": (i32, (vp, vp, vp, vp, sz, sz, sz, f32, vp, dbl_p) + _ERR),
    "h3_cuda_sdpa_f16_dev": (i32, (vp, vp, vp, vp, sz, sz, sz, f32, vp, dbl_p) + _ERR),
    "h3_cuda_sdpa_f16_dev_ex": (i32, (vp, vp, vp, vp, sz, sz, sz, f32, i32, vp, dbl_p, cs, sz) + _ERR),
    "h3_cuda_qkv_rope_sdpa_f16_dev": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f32, f32, i32, vp, dbl_p, dbl_p,
                                            cs, sz) + _ERR),
    "h3_cuda_sdpa_backend_name": (cs, ()),
    "h3_cuda_sdpa_last_backend_name": (cs, ()),
    "h3b_sdpa_bf16_dev": (i32, (vp, vp, sz, vp, sz, vp, sz, sz, sz, sz, sz, f32, vp, sz) + _ERR),
    "h3_cuda_adaln_f32": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, sz, f32, vp, dbl_p) + _ERR),
    "h3_cuda_gate_f32": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, vp, dbl_p) + _ERR),
    "h3_cuda_swiglu_f32": (i32, (vp, vp, sz, sz, vp, dbl_p) + _ERR),
    "h3_cuda_qkv_rope_f32": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f32, vp, vp, vp, dbl_p) + _ERR),
    "h3_cuda_nvfp4_sf_bytes": (sz, (sz, sz)),
    "h3_cuda_quantize_act_nvfp4_dev": (i32, (vp, vp, sz, sz, vp, vp) + _ERR),
    "h3b_adaln_project_dev": (i32, (vp, vp, vp, sz, sz, vp, vp) + _ERR),
    "h3_cuda_gemm_f32_dd": (i32, (vp, vp, vp, sz, sz, sz, vp, dbl_p) + _ERR),
    "h3_cuda_bias_add_f32_dev": (i32, (vp, vp, vp, sz, sz) + _ERR),
    "h3_cuda_gemm_f32_dd_ex": (i32, (vp, vp, vp, sz, sz, sz, vp, f32, f32, dbl_p) + _ERR),
    "h3_cuda_gemm_f32_dd_tf32_ex": (i32, (vp, vp, vp, sz, sz, sz, vp, f32, f32) + _ERR),
    "h3b_dense_f32_dev": (i32, (vp, vp, vp, vp, sz, sz, sz, vp) + _ERR),
    "h3b_final_head_scratch_bytes": (sz, (sz, sz)),
    "h3b_final_head_f32_dev": (i32, (vp, vp, vp, vp, sz, sz, vp, vp, sz, f32, vp, sz, vp) + _ERR),
    "h3b_euler_step_f32_dev": (i32, (vp, vp, vp, sz, f32, f32) + _ERR),
    "h3b_dit_create": (vp, (vp, C.POINTER(DitConfig)) + _ERR),
    "h3b_dit_free": (None, (vp,)),
    "h3b_ckpt_open": (vp, (C.c_char_p,) + _ERR),
    "h3b_ckpt_close": (None, (vp,)),
    "h3b_ckpt_count": (sz, (vp,)),
    "h3b_ckpt_get": (i32, (vp, sz, vp)),
    "h3b_ckpt_find": (i32, (vp, C.c_char_p, vp)),
    "h3b_dit_load_int8_convrot_block": (i32, (vp, vp, C.c_uint, C.c_uint) + _ERR),
    "h3b_gemm_i8_plan": (i32, (sz, sz, sz, i32, sz) + (C.POINTER(i32),) * 7),
    "h3b_dit_load_w4a8_block": (i32, (vp, vp, C.c_uint, C.c_uint) + _ERR),
    "h3b_dit_load_nvfp4_block": (i32, (vp, vp, C.c_uint, C.c_uint, C.c_uint) + _ERR),
    "h3b_dit_set_linear": (i32, (vp, C.c_uint, i32, vp) + _ERR),
    "h3b_dit_set_linear_nvfp4": (i32, (vp, C.c_uint, i32, vp) + _ERR),
    "h3b_dit_set_block_aux": (i32, (vp, C.c_uint, vp, vp, vp, vp, vp) + _ERR),
    "h3b_dit_set_adaln": (i32, (vp, C.c_uint, vp, vp) + _ERR),
    "h3b_dit_project_modulation": (i32, (vp, vp) + _ERR),
    "h3b_dit_modulation": (vp, (vp, C.c_uint)),
    "h3b_dit_reserve": (i32, (vp, sz, sz) + _ERR),
    "h3b_dit_block_forward_dev": (i32, (vp, C.c_uint, vp, sz, vp, vp, vp, vp, vp, sz, vp) + _ERR),
    "h3b_dit_layers_forward_dev": (i32, (vp, C.c_uint, C.c_uint, vp, sz, vp, vp, vp, vp, sz, vp) + _ERR),
    "h3b_dit_layers_forward_graph_dev": (i32, (vp, C.c_uint, C.c_uint, vp, sz, vp, vp, vp, vp, sz, vp) + _ERR),
    "h3b_dit_graph_nodes": (sz, (vp,)),
    "h3b_dit_layers_forward_f32": (i32, (vp, C.c_uint, C.c_uint, vp, vp, sz, vp, vp, vp, vp, sz, vp) + _ERR),
    "h3b_dit_launches_per_block": (i32, (vp,)),
    "h3_cuda_gemm_fp4_bs_dev": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, vp, dbl_p) + _ERR),
    "h3b_w4g_exact_weight_create": (i32, (vp, vp, vp, sz, sz, C.POINTER(vp)) + _ERR),
    "h3b_w4g_exact_weight_free": (None, (vp,)),
    "h3b_gemm_w4g_exact_dev": (i32, (vp, vp, vp, vp, sz, vp, i32) + _ERR),
    "h3b_gemm_fp4_dev": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, f32, vp, i32) + _ERR),
    "h3b_gemm_fp4_w_preq_dev": (i32, (vp, vp, vp, vp, sz, f32, i32, vp, vp, vp, sz, sz, vp, i32) + _ERR),
    "h3b_gemm_fp4_w_preq_qkv_rope_dev": (i32, (vp, vp, vp, vp, sz, f32, vp, vp, vp, vp, sz, sz, f32, vp, vp, vp) + _ERR),
    "h3b_gemm_fp4_swiglu_dev": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, f32, vp, i32) + _ERR),
    "h3_cuda_nvfp4_weight_create": (i32, (vp, vp, vp, f32, sz, sz, C.POINTER(vp), dbl_p) + _ERR),
    "h3_cuda_nvfp4_weight_ensure_ready": (i32, (vp,) + _ERR),
    "h3_cuda_nvfp4_weight_free": (None, (vp, vp)),
    "h3_cuda_nvfp4_weight_packed": (vp, (vp,)),
    "h3_cuda_nvfp4_weight_sf": (vp, (vp,)),
    "h3_cuda_nvfp4_weight_scale2": (f32, (vp,)),
    "h3_cuda_nvfp4_weight_n": (sz, (vp,)),
    "h3_cuda_nvfp4_weight_k": (sz, (vp,)),
    "h3_cuda_nvfp4_gemm_scratch_bytes": (sz, (sz, sz, sz)),
    "h3_cuda_gemm_fp4_w_act_dev": (i32, (vp, vp, vp, f32, sz, vp, vp, dbl_p, dbl_p) + _ERR + (cs,)),
    "h3_cuda_gemm_fp4_w_act_dev_swiglu": (i32, (vp, vp, vp, f32, sz, vp, vp, vp, dbl_p, dbl_p) + _ERR + (cs,)),
    "h3_cuda_gemm_fp4_w_act_dev_gate": (i32, (vp, vp, vp, f32, sz, vp, vp, vp, sz, sz, vp, vp, vp, dbl_p, dbl_p) + _ERR + (cs,)),
    "h3_ulysses_comm_init": (i32, (C.POINTER(UlyssesCfg), C.POINTER(i32), i32) + _ERR),
    "h3_ulysses_comm_destroy": (None, (C.POINTER(UlyssesCfg),)),
    "h3_ulysses_comm_bind": (i32, (C.POINTER(UlyssesCfg), i32, vp, vp) + _ERR),
    "h3_ulysses_comm_set_compute": (i32, (C.POINTER(UlyssesCfg), i32, vp) + _ERR),
    "h3_ulysses_a2a_qkv": (i32, (C.POINTER(UlyssesCfg), vp, vp, sz, sz, sz, i32) + _ERR),
    "h3_ulysses_a2a_attn_out": (i32, (C.POINTER(UlyssesCfg), vp, vp, sz, sz, sz, i32) + _ERR),
    "h3b_ulysses_unique_id": (i32, (vp,) + _ERR),
    "h3b_ulysses_comm_init_rank": (i32, (C.POINTER(UlyssesCfg), i32, i32, vp, i32) + _ERR),
    "h3b_dit_set_ulysses": (i32, (vp, C.POINTER(UlyssesCfg)) + _ERR),
    "h3b_ulysses_direct_setup": (i32, (C.POINTER(UlyssesCfg), sz, sz, sz) + _ERR),
    "h3b_ulysses_setup_protocol": (i32, (vp,)),
    "h3b_ulysses_direct_get": (vp, (C.POINTER(UlyssesCfg),)),
    "h3b_ulysses_direct_enable": (None, (C.POINTER(UlyssesCfg), i32)),
    "h3b_ulysses_barrier": (i32, (C.POINTER(UlyssesCfg),) + _ERR),
    "h3b_ulysses_check": (i32, (C.POINTER(UlyssesCfg), C.POINTER(C.c_int)) + _ERR),
    "h3b_ulysses_barrier_selftest": (i32, (C.c_longlong, C.POINTER(C.c_int), C.POINTER(C.c_int)) + _ERR),
    "h3b_sdpa_bf16_scatter_dev": (i32, (vp, vp, sz, f32) + _ERR),
    "h3b_dit_layers_forward_ulysses_dev": (i32, (vp, C.c_uint, C.c_uint, vp, sz, sz, vp, vp, vp, vp, sz, vp) + _ERR),
    "h3b_dit_layers_forward_ulysses_f32": (i32, (vp, C.c_uint, C.c_uint, vp, vp, sz, sz, vp, vp, vp, vp, sz, vp) + _ERR),
    "h3_dit_w4a8_fill_metal_video_pos": (i32, (sz, i32, i32, i32, vp, vp, vp) + _ERR),
    "h3_dit_w4a8_video_span_sum": (f32, (i32,)),
    "h3_dit_w4a8_rope_tables_f32": (i32, (vp, sz, vp, vp, vp, f32, vp, vp) + _ERR),
    "h3_dit_w4a8_t_row_from_sigma": (sz, (f32, sz)),
    "h3b_dit_video_rope_tables": (i32, (vp, sz, i32, i32, i32, f32, sz, vp, vp) + _ERR),
    # ---- the rest of the reference's operator surface
    "h3_cuda_copy_stream_synchronize": (i32, (vp,) + _ERR),
    "h3_cuda_cublas_use_side": (i32, (vp, i32) + _ERR),
    "h3_cuda_cublas_stream": (vp, (vp,)),
    "h3_cuda_recreate_blas": (i32, (vp,) + _ERR),
    "h3_cuda_dit_scratch_rehome": (i32, (vp,) + _ERR),
    "h3_cuda_dit_scratch_check": (i32, (vp,) + _ERR),
    "h3_cuda_host_register": (i32, (vp, sz) + _ERR),
    "h3_cuda_host_unregister": (None, (vp,)),
    "h3_cuda_gemm_f32": (i32, (vp, vp, vp, sz, sz, sz, vp, dbl_p) + _ERR),
    "h3_cuda_gemm_f32_dw": (i32, (vp, vp, vp, sz, sz, sz, vp, dbl_p) + _ERR),
    "h3_cuda_gemm_f32in_f16w_f32out_dd_ex": (i32, (vp, vp, vp, sz, sz, sz, vp, f32, f32) + _ERR),
    "h3_cuda_convrot_act_f16_dd": (i32, (vp, vp, sz, sz, i32, vp) + _ERR),
    "h3_cuda_epi_fuse_ink_prep_fc2": (i32, (vp, vp, sz, sz, i32, C.POINTER(vp), C.POINTER(vp)) + _ERR),
    "h3_cutlass_nvfp4_fc1_f32_run": (i32, (vp, vp, vp, vp, vp, sz, sz, sz, vp, dbl_p) + _ERR),
    "h3_nvfp4_swiglu_requant_dev": (i32, (vp, vp, f32, vp, sz, sz, vp, vp) + _ERR),
    "h3_cuda_nvfp4_chain_scratch_bytes": (sz, (sz, sz, sz)),
    "h3_cuda_gemm_fp4_pre_q_dev": (i32, (vp, vp, vp, vp, sz, vp, vp, vp, sz, sz, vp, vp, vp, dbl_p) + _ERR + (cs,)),
    "h3_nvfp4_debug_nan_dev": (i32, ()),
    "h3_nvfp4_debug_scan_dev": (None, (vp, vp, sz, cs, cs, cs)),
    "h3_cuda_sdpa_f32": (i32, (vp, vp, vp, vp, sz, sz, sz, f32, vp, dbl_p) + _ERR),
    "h3_cuda_sdpa_f16": (i32, (vp, vp, vp, vp, sz, sz, sz, f32, vp, dbl_p) + _ERR),
    "h3_cuda_sdpa_f16_ex": (i32, (vp, vp, vp, vp, sz, sz, sz, f32, i32, vp, dbl_p, cs, sz) + _ERR),
    "h3_cuda_qkv_rope_sdpa_f16_dev_layout": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f32, f32, i32, i32, i32, vp,
                                                   dbl_p, dbl_p, cs, sz) + _ERR),
    "h3_cuda_qkv_rope_sdpa_f16_dev_layout_f16qkv": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f32, f32, i32, i32, i32,
                                                          vp, dbl_p, dbl_p, cs, sz) + _ERR),
    "h3_cuda_qkv_rope_sdpa_f16_dev_f16qkv": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, f32, f32, i32, vp, dbl_p, dbl_p,
                                                   cs, sz) + _ERR),
    "h3_cuda_sdpa_bind_kvcat": (None, (vp, vp, sz)),
    "h3_cuda_sdpa_bind_kvsave": (None, (vp, vp, vp, sz)),
    "h3_cuda_sdpa_clear_kvext": (None, ()),
    "h3_cuda_token_pool_f32": (i32, (vp, vp, sz, vp, vp, sz, sz, sz, vp, C.POINTER(vp), C.POINTER(vp), dbl_p) + _ERR),
    "h3_cuda_token_expand_f32": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, C.c_uint32, C.c_uint32, f32, vp, dbl_p) + _ERR),
    "h3_cuda_token_pool_f32_dev": (i32, (vp, vp, sz, vp, vp, sz, sz, sz, vp, vp, vp, dbl_p) + _ERR),
    "h3_cuda_token_expand_f32_dev": (i32, (vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, C.c_uint32, C.c_uint32, f32, vp, dbl_p) + _ERR),
    "h3_cuda_dist_attn_configure": (i32, (vp, sz, sz, sz, i32, i32, i32, f32, f32, i32) + _ERR),
    "h3_cuda_dist_attn_clear": (None, ()),
    "h3_cuda_dist_attn_active": (i32, ()),
    "h3_cuda_sol_cute_set_step": (None, (i32,)),
    "h3_cuda_sol_profile_add_unpack": (None, (C.c_double,)),
    "h3_cuda_sage3_pool_bytes": (sz, ()),
    "h3_nvfp4_cuda_enabled": (i32, ()),
    "h3_nvfp4_cuda_cache_clear": (None, ()),
    "h3_nvfp4_cuda_encode_text_layers": (i32, (vp, vp, sz, C.c_uint) + _ERR),
    "h3_nvfp4_cuda_gqa_causal": (i32, (vp, vp, vp, sz, sz, sz, sz, vp) + _ERR),
    "h3b_sdpa_strided_dev": (i32, (vp, i32, vp, sz, sz, vp, sz, sz, vp, sz, sz, sz, sz, sz, sz, f32, vp, sz, sz) + _ERR),
    "h3_dit_patchify_video": (i32, (vp, i32, i32, i32, i32, vp, sz)),
    "h3_dit_unpatchify_video": (i32, (vp, i32, i32, i32, i32, vp, sz)),
    "h3_dit_pack_audio": (i32, (vp, i32, i32, vp, sz)),
    "h3_dit_unpack_audio": (i32, (vp, i32, i32, vp, sz)),
    "h3_dit_reuse_schedule": (i32, (i32, i32, vp, sz)),
    "h3_dit_forward": (i32, (vp, i32, vp, vp, vp, vp) + _ERR),
    "h3_dit_denoise_euler": (i32, (vp, vp, vp, i32, vp, vp) + _ERR),
    "h3_dit_video_elements": (sz, (vp,)),
    "h3_dit_audio_elements": (sz, (vp,)),
    "h3_dit_free": (None, (vp,)),
    "h3b_plugin_count": (sz, ()),
    "h3b_plugin_get": (i32, (sz, C.POINTER(cs), C.POINTER(cs), C.POINTER(cs), C.POINTER(cs))),
    "h3b_plugin_value": (cs, (cs,)),
    "h3b_plugin_enabled": (i32, (cs,)),
    "h3_ulysses_validate": (i32, (i32, i32, i32, i32, i32) + _ERR),
    "h3_ulysses_pad_seq": (sz, (sz, i32)),
    "h3_ulysses_local_rows": (sz, (sz, i32, i32)),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once; raises if it was not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise H3Error(f"{LIB_PATH} is missing: run `python -m h3c_b200.build` (there is no fallback path)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = list(args)
        _lib = lib
    return _lib


def declared_symbols():
    return sorted(_SIGS)


def ptr(t) -> int | None:
    """Raw device (or host) address of a torch tensor / numpy array; None passes NULL."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    if hasattr(t, "ctypes"):
        return t.ctypes.data
    return int(t)


def call(name: str, *args):
    """Calls an entry point that ends in (error, error_size) and returns 1/0; raises H3Error on 0."""
    lib = load()
    err = C.create_string_buffer(ERR_LEN)
    rc = getattr(lib, name)(*args, err, ERR_LEN)
    if rc != 1:
        raise H3Error(f"{name}: {err.value.decode(errors='replace') or 'failed'}")
    return rc
