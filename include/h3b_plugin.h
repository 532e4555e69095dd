/* Switch registry of libh3_b200: every environment switch the library (or its bench) reads is listed here with
 * its status, stage and default, and is read through h3_plugin_value / h3_plugin_enabled, never through a bare
 * getenv.  Same record type, same three functions and the same X-macro catalogue as the reference's registry
 * (tools/h3_plugin.h:24-239: h3_plugin_def {name, status, stage, default_value}, H3_PLUGIN_BUILTIN_DEFS,
 * h3_plugin_find, h3_plugin_enabled), so a tree that carries both can merge the two catalogues by
 * concatenating the X(...) lines; tests/test_plugin_registry.py restates the reference's lint
 * (tools/check_plugin_registry.sh:1-72) over this repository's sources.
 *
 * Status: STABLE (product path) or EXPERIMENTAL (A/B or diagnosis only).  Stage: DIT, SP (sequence
 * parallelism), MISC.  Default "0" = off, "1" = on, anything else is a value.
 */
#ifndef H3B_PLUGIN_H
#define H3B_PLUGIN_H

#include <stdlib.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

#define H3_PLUGIN_BUILTIN_DEFS(X)                                                                              \
    /* this library's own switches */                                                                          \
    X("H3B_GEMM_PAIRS", "STABLE", "DIT", "1")        /* 0: int8 GEMM on single-CTA tiles instead of CTA pairs */ \
    X("H3B_GEMM_SPLITK", "STABLE", "DIT", "1")       /* 0: whole tiles only; n >= 2: n slices of K per tail tile */ \
    X("H3B_FP4_WIDE", "STABLE", "DIT", "1")          /* 0: NVFP4 GEMM on 128 x 128 tiles */                     \
    X("H3B_FP4_QKV_ROPE", "STABLE", "DIT", "1")      /* 0: NVFP4 QKV projection, then stand-alone QK-norm + RoPE */ \
    X("H3B_FP4_PAIRS", "STABLE", "DIT", "1")         /* 0: NVFP4 GEMM on single CTAs, no 256 x 256 pair tiles */ \
    X("H3B_ATTN_EMU", "STABLE", "DIT", "12")         /* attention kernel variant: 12, 13, 10, 0; 212, 213 = CTA pairs */ \
    X("H3B_ULYSSES_BARRIER", "STABLE", "SP", "flag") /* flag | nccl: barrier of the exchange-free form */       \
    X("H3B_ULYSSES_DIRECT", "STABLE", "SP", "1")     /* 0: NCCL exchange instead of direct peer stores (bench) */ \
    /* switches of the reference that this library honours with the reference's meaning */                     \
    X("H3_CONVROT_SYLVESTER", "EXPERIMENTAL", "DIT", "0") /* 1: Walsh-Hadamard (radix-2) ConvRot, h3_w4a8_dequant.c:371 */ \
    X("H3_DIT_QKV_GROUPED", "EXPERIMENTAL", "DIT", "0")                                                        \
    X("H3_DIT_ROPE_HALF_OFFSET", "EXPERIMENTAL", "DIT", "0")                                                   \
    X("H3_DIT_ROPE_SPLIT_HALF", "EXPERIMENTAL", "DIT", "1")                                                    \
    X("H3_DIT_T_ROW_BY_SIGMA", "EXPERIMENTAL", "DIT", "0")                                                     \
    X("H3_NVFP4_DEBUG_NAN", "EXPERIMENTAL", "DIT", "0")

typedef struct {
    const char *name;
    const char *status;
    const char *stage;
    const char *default_value;
} h3_plugin_def;

#define H3_PLUGIN_DEF_ITEM(n, s, g, d) {n, s, g, d},
static const h3_plugin_def h3_plugin_builtins[] = {H3_PLUGIN_BUILTIN_DEFS(H3_PLUGIN_DEF_ITEM)};
#undef H3_PLUGIN_DEF_ITEM

#if defined(__GNUC__)
__attribute__((unused))
#endif
static const size_t h3_plugin_builtin_count = sizeof(h3_plugin_builtins) / sizeof(h3_plugin_builtins[0]);

static inline const h3_plugin_def *h3_plugin_find(const char *name) {
    size_t i;
    if (!name) return NULL;
    for (i = 0; i < h3_plugin_builtin_count; i++)
        if (strcmp(h3_plugin_builtins[i].name, name) == 0) return &h3_plugin_builtins[i];
    return NULL;
}

/* Addition: the value of a switch, i.e. the environment's if set and not empty, else the catalogue default;
 * NULL for a name that is not registered (reading an unregistered switch is a bug the lint catches). */
static inline const char *h3_plugin_value(const char *name) {
    const h3_plugin_def *def = h3_plugin_find(name);
    const char *e;
    if (!def) return NULL;
    e = getenv(name);
    return (e && e[0]) ? e : def->default_value;
}

static inline int h3_plugin_enabled(const char *name) {
    const char *val = h3_plugin_value(name);
    if (!val || !val[0]) return 0;
    return strcmp(val, "0") != 0 && strcmp(val, "false") != 0 && strcmp(val, "off") != 0 && strcmp(val, "no") != 0;
}

#ifdef __cplusplus
}
#endif

#endif
