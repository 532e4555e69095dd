/* Exports the reference's header-only (static inline) epilogue formulas as
 * linkable symbols so the test-suite can call them through ctypes.
 * Compiled only into oracle/_ref/libh3_ref.so, with -I pointing at the h3.c
 * tree; nothing from that tree is copied here.  TEST INFRASTRUCTURE ONLY. */
#include "h3_dit_act_f16.h"
#include "h3_dit_fused_epi.h"
#include "h3_dit_int8_opt.h"

void ref_gate_adaln_f32(const float *residual, const float *branch, const float *norm_w,
                        const float *modulation, const uint32_t *row_map, size_t rows,
                        size_t width, size_t slots, size_t gate_slot, size_t shift_slot,
                        size_t scale_slot, float epsilon, float *gated, float *normed) {
    h3_dit_gate_adaln_f32(residual, branch, norm_w, modulation, row_map, rows, width, slots,
                          gate_slot, shift_slot, scale_slot, epsilon, gated, normed);
}

void ref_dequant_swiglu_f32(const int32_t *acc, const float *act_scales, int per_tensor,
                            const float *s_channel, size_t rows, size_t width,
                            const float *lora, float *out) {
    h3_dit_dequant_swiglu_f32(acc, act_scales, per_tensor, s_channel, rows, width, lora, out);
}

void ref_dequant_gate_f32(const int32_t *acc, const float *act_scales, int per_tensor,
                          const float *s_channel, const float *residual,
                          const float *modulation, const uint32_t *row_map, size_t rows,
                          size_t width, size_t slots, size_t gate_slot, const float *lora,
                          float *out) {
    h3_dit_dequant_gate_f32(acc, act_scales, per_tensor, s_channel, residual, modulation,
                            row_map, rows, width, slots, gate_slot, lora, out);
}

float ref_act_f16_pre_scale(float absmax, int gs) { return h3_dit_act_f16_pre_scale(absmax, gs); }

size_t ref_int8_gemm_tile_rows(size_t m, size_t n) { return h3_dit_int8_gemm_tile_rows(m, n); }
