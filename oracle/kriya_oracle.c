/*
 * CPU oracle for the KriyaRT paged KV-cache hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C and fp32, the arithmetic of the reference's
 * Metal kernels and of the scalar CPU loops inside the reference's own tests.
 * It is the checker the CUDA kernels are compared against and the timed CPU
 * baseline of the benchmark.  Nothing in the shipped library links, loads or
 * calls it; only the test-suite, the smoke check and the benchmark's CPU
 * baseline leg may do so.
 *
 * Parity status: the reference is Rust + Metal and can be neither compiled nor
 * run in this environment.  Pinning therefore rests on (a) the literal golden
 * arrays of the reference's bookkeeping tests (covered by the Python
 * bookkeeping oracle next to this file) and (b) for the numerics, on the
 * closed-form inputs, CPU loops and tolerances of the reference's kernel tests,
 * which are restated below (ko_ref_test_*) and compared with the kernel-math
 * restatement.  The reference holds no literal output vectors for the
 * numerics, so those are pinned to formulas, not to stored numbers.  Not pinned
 * by any reference test ("parity unpinned" there): the split-K merge on device,
 * the copy-on-write data copy, prefill with a non-zero prefix, fp16 storage.
 *
 * Every function cites the reference lines it follows:
 *   metal: = kernels/metal/paged_gqa_and_deltanet.metal
 *   enc:   = crates/kriya-backend-metal/src/encoder.rs
 *   tsc:   = crates/kriya-backend-metal/tests/test_shader_compile.rs
 *   rwv:   = crates/kriya-backend-metal/tests/real_world_validation.rs
 *   quant: = crates/kriya-core/src/quantizer.rs
 *
 * Build: gcc -O3 -march=native -ffp-contract=off -fopenmp -shared -fPIC
 * (-ffp-contract=off keeps every fma() explicit, as the shader source has it).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define KO_EXPORT __attribute__((visibility("default")))

/* ---- parameter blocks, byte-identical to enc:159-187 / metal:60-85 ---------- */
typedef struct {
    uint32_t num_q_heads, num_kv_heads, head_dim, rotary_dim, block_size_tokens, apply_qk_norm;
    float rms_eps, rope_theta;
    uint32_t max_seq_len, has_table, _pad0, _pad1;
} ko_rope_params; /* RopeKvWriteParams, 48 bytes */

typedef struct {
    uint32_t num_q_heads, num_kv_heads, head_dim, block_size_tokens, max_split_k_tiles, max_query_tokens;
    float sm_scale, logit_softcap;
} ko_gqa_params; /* BsrGqaParams, 32 bytes */

typedef struct {
    uint32_t request_idx, kv_block_start, kv_block_count, is_split_k;
} ko_tile; /* CtaWorkTile, crates/kriya-kv/src/bsr_paged.rs:285-297 */

enum { KO_BF16 = 0, KO_FP16 = 1 };

/* ---- 16-bit storage --------------------------------------------------------- */

/* metal:95-97, quant:26-29 */
static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* metal:99-103, quant:19-24: round to nearest even on the bit pattern, no NaN case */
static inline uint16_t f32_to_bf16(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    uint32_t lsb = (u >> 16) & 1u;
    return (uint16_t)((u + 0x7FFFu + lsb) >> 16);
}

/* IEEE binary16 <-> binary32, round to nearest even.  The reference has no fp16
 * storage path (its kernels treat all storage as bf16 bit patterns); fp16 is the
 * same math with this storage rounding instead. */
static inline float fp16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | (man << 13);
    } else {
        u = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_fp16(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t abs = u & 0x7FFFFFFFu;
    if (abs >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((abs > 0x7F800000u) ? 0x200u : 0u));
    }
    if (abs >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (abs < 0x33000001u) { /* below half of the smallest subnormal */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(abs >> 23) - 127;
    uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_bits;
    if (e < -14) { /* subnormal result */
        shift = (uint32_t)(13 + (-14 - e));
        half_bits = 0;
    } else {
        shift = 13;
        half_bits = (uint32_t)(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t)(sign | (half_bits + q)); /* carry into the exponent is correct by construction */
}

static inline float load16(uint16_t b, int dtype) { return dtype == KO_FP16 ? fp16_to_f32(b) : bf16_to_f32(b); }
static inline uint16_t store16(float v, int dtype) { return dtype == KO_FP16 ? f32_to_fp16(v) : f32_to_bf16(v); }

KO_EXPORT void ko_f32_to_16(const float* src, uint16_t* dst, size_t n, int dtype) {
    for (size_t i = 0; i < n; ++i) dst[i] = store16(src[i], dtype);
}
KO_EXPORT void ko_16_to_f32(const uint16_t* src, float* dst, size_t n, int dtype) {
    for (size_t i = 0; i < n; ++i) dst[i] = load16(src[i], dtype);
}

/* A 32-lane sum.  The shader calls simd_sum (metal:154,307,376,449); the hardware's
 * association order is not documented, so a butterfly (xor 16,8,4,2,1) is used. */
static inline float simd_sum32(float lane[32]) {
    for (int off = 16; off >= 1; off >>= 1)
        for (int i = 0; i < off; ++i) lane[i] = lane[i] + lane[i + off];
    return lane[0];
}

static inline float clampf(float x, float lo, float hi) { return x < lo ? lo : (x > hi ? hi : x); }
/* metal:105-107 */
static inline float safe_tanh(float x) { return tanhf(clampf(x, -15.0f, 15.0f)); }

/* ---- RoPE table ------------------------------------------------------------- */

/* enc:1939-1950: table[pos][pair] = (cos, sin) of pos * theta^-(2*pair/rotary_dim), all in f32 */
KO_EXPORT void ko_rope_table(float* table, uint32_t max_seq_len, uint32_t rotary_dim, float theta) {
    uint32_t half_rot = rotary_dim / 2u;
    if (half_rot < 1u) half_rot = 1u;
    for (uint32_t pos = 0; pos < max_seq_len; ++pos) {
        for (uint32_t i = 0; i < half_rot; ++i) {
            float freq_exp = (2.0f * (float)i) / (float)rotary_dim;
            float inv_freq = powf(theta, -freq_exp);
            float angle = (float)pos * inv_freq;
            table[((size_t)pos * half_rot + i) * 2 + 0] = cosf(angle);
            table[((size_t)pos * half_rot + i) * 2 + 1] = sinf(angle);
        }
    }
}

/* ---- DType::Q4KvGroup32: the 4-bit KV-cache format ----------------------------- */

/* crates/kriya-core/src/tensor.rs:50-51,77,91: 32 values -> 16 bytes of 4-bit codes + f16 scale + f16 min = 20 bytes
 * ("FlexGen-style 4-bit KV cache / activation group-32 compression"), switched on by compress_kv_cache_q4
 * (crates/kriya-core/src/hardware.rs:57,159-165).  The reference declares the format and ships neither a quantiser
 * nor a kernel for it.  Its arithmetic is restated here from the reference's own 4-bit affine group quantiser, the only
 * one of that family it implements (quantize_f32_to_q4_group64 / dequantize, crates/kriya-core/src/quantizer.rs:61-127),
 * with the group size and header type of this format: min and max of the group, range = max(max - min, 1e-8),
 * scale = range / 15, bias = min, both rounded to the header's storage type (f16 here, bf16 there); the codes are taken
 * with the ROUNDED scale (floored at 1e-8) and bias, q = clamp(round((v - bias) / scale), 0, 15) with round-half-away
 * (f32::round); value 2i sits in the low nibble of byte i, value 2i + 1 in the high nibble; a value is restored as
 * fma(q, scale, bias).  Block layout: bytes 0..15 codes, 16..17 scale, 18..19 min (little endian).
 * A cache row of D values is D / 32 consecutive blocks; the pool keeps the [block][token][head] order of the 16-bit pool. */
#define KO_Q4_GROUP 32u
#define KO_Q4_BLOCK_BYTES 20u

KO_EXPORT void ko_q4kv_quantize(const float* v, uint32_t n_groups, uint8_t* out) {
    for (uint32_t g = 0; g < n_groups; ++g) {
        const float* x = v + (size_t)g * KO_Q4_GROUP;
        uint8_t* b = out + (size_t)g * KO_Q4_BLOCK_BYTES;
        float mn = INFINITY, mx = -INFINITY;
        for (uint32_t i = 0; i < KO_Q4_GROUP; ++i) {
            mn = fminf(mn, x[i]);
            mx = fmaxf(mx, x[i]);
        }
        const float range = fmaxf(mx - mn, 1e-8f);
        const uint16_t scale16 = f32_to_fp16(range / 15.0f), min16 = f32_to_fp16(mn);
        const float eff_scale = fmaxf(fp16_to_f32(scale16), 1e-8f), eff_min = fp16_to_f32(min16);
        for (uint32_t i = 0; i < KO_Q4_GROUP / 2u; ++i) {
            const float q0 = clampf(roundf((x[2 * i] - eff_min) / eff_scale), 0.0f, 15.0f);
            const float q1 = clampf(roundf((x[2 * i + 1] - eff_min) / eff_scale), 0.0f, 15.0f);
            b[i] = (uint8_t)(((uint8_t)q0 & 0x0Fu) | (((uint8_t)q1 & 0x0Fu) << 4));
        }
        b[16] = (uint8_t)(scale16 & 0xFFu);
        b[17] = (uint8_t)(scale16 >> 8);
        b[18] = (uint8_t)(min16 & 0xFFu);
        b[19] = (uint8_t)(min16 >> 8);
    }
}

static inline float q4kv_value(const uint8_t* pool, size_t elem) {
    const uint8_t* b = pool + (elem / KO_Q4_GROUP) * KO_Q4_BLOCK_BYTES;
    const uint32_t i = (uint32_t)(elem % KO_Q4_GROUP);
    const uint32_t q = (i & 1u) ? (uint32_t)(b[i >> 1] >> 4) : (uint32_t)(b[i >> 1] & 0x0Fu);
    const float scale = fp16_to_f32((uint16_t)(b[16] | (b[17] << 8))), mn = fp16_to_f32((uint16_t)(b[18] | (b[19] << 8)));
    return fmaf((float)q, scale, mn);
}

KO_EXPORT void ko_q4kv_dequantize(const uint8_t* in, uint32_t n_groups, float* out) {
    for (size_t e = 0; e < (size_t)n_groups * KO_Q4_GROUP; ++e) out[e] = q4kv_value(in, e);
}

/* Cache format of every following append / decode / prefill call of the oracle: 0 = 16-bit pool (uint16 per element),
 * 1 = Q4KvGroup32 pool (the cache pointers are then byte arrays of 20-byte blocks in element order). */
static int g_kv_q4 = 0;
KO_EXPORT void ko_set_kv_format(int q4) { g_kv_q4 = q4; }

/* One cached element by its index in [block][token][head][d] order. */
static inline float kv_elem(const uint16_t* pool, size_t elem, int dtype) {
    return g_kv_q4 ? q4kv_value((const uint8_t*)pool, elem) : load16(pool[elem], dtype);
}

/* ---- fused QK-norm + RoPE + KV append --------------------------------------- */

/* metal:115-226, one (token, head) at a time in the shader's lane order.
 * q_inout [T,Hq,D] is rotated in place, K is rotated into its cache slot, V is copied
 * bit for bit.  The slot is (page_indices[indptr[r+1]-1], last_page_len[r]-1). */
KO_EXPORT void ko_rope_kv_append(uint16_t* q_inout, const uint16_t* k_in, const uint16_t* v_in,
                                 const uint16_t* q_norm_w, const uint16_t* k_norm_w, uint16_t* cache_k,
                                 uint16_t* cache_v, const int32_t* indptr, const int32_t* indices,
                                 const int32_t* last_len, const uint32_t* positions, uint32_t num_tokens,
                                 const ko_rope_params* p, const float* cos_sin_table, int dtype) {
    const uint32_t D = p->head_dim, Hq = p->num_q_heads, Hkv = p->num_kv_heads;
    const uint32_t half_rot = p->rotary_dim / 2u, half_d = D / 2u;
    const int do_norm = p->apply_qk_norm != 0u;
#pragma omp parallel for schedule(static)
    for (int64_t job = 0; job < (int64_t)num_tokens * (Hq + Hkv); ++job) {
        const uint32_t r = (uint32_t)(job / (Hq + Hkv));
        const uint32_t head = (uint32_t)(job % (Hq + Hkv));
        const int is_q = head < Hq;
        const uint32_t lh = is_q ? head : head - Hq;
        const float pos = (float)positions[r];
        const uint16_t* src = is_q ? q_inout + ((size_t)r * Hq + lh) * D : k_in + ((size_t)r * Hkv + lh) * D;

        float rms_scale = 1.0f;
        if (do_norm) { /* metal:145-158 */
            float lane[32];
            for (uint32_t l = 0; l < 32; ++l) {
                float s = 0.0f;
                for (uint32_t d = l; d < D; d += 32u) {
                    float v = load16(src[d], dtype);
                    s = fmaf(v, v, s);
                }
                lane[l] = s;
            }
            float sum_sq = simd_sum32(lane);
            rms_scale = 1.0f / sqrtf(sum_sq / (float)D + p->rms_eps);
        }
        float k_row[256], v_row[256]; /* the rotated key and the value of this (token, head) before they are stored */
        size_t dst = 0;
        if (!is_q) { /* metal:162-167 */
            int32_t last_ptr = indptr[r + 1] - 1;
            uint32_t blk = (uint32_t)indices[last_ptr];
            uint32_t slot = (uint32_t)(last_len[r] - 1);
            dst = (((size_t)blk * p->block_size_tokens + slot) * Hkv + lh) * D;
        }
        for (uint32_t i = 0; i < half_d; ++i) { /* metal:171-225 */
            const uint32_t d0 = i, d1 = i + half_d;
            float x0 = load16(src[d0], dtype) * rms_scale;
            float x1 = load16(src[d1], dtype) * rms_scale;
            if (do_norm) {
                const uint16_t* w = is_q ? q_norm_w : k_norm_w;
                x0 *= load16(w[d0], dtype);
                x1 *= load16(w[d1], dtype);
            }
            if (i < half_rot) {
                float c, s;
                if (p->has_table != 0u && (uint32_t)pos < p->max_seq_len && cos_sin_table != NULL) {
                    c = cos_sin_table[((size_t)(uint32_t)pos * half_rot + i) * 2 + 0];
                    s = cos_sin_table[((size_t)(uint32_t)pos * half_rot + i) * 2 + 1];
                } else {
                    float freq_exp = (float)(2u * i) / (float)p->rotary_dim;
                    float inv_freq = powf(p->rope_theta, -freq_exp);
                    float angle = pos * inv_freq;
                    c = cosf(angle);
                    s = sinf(angle);
                }
                float rot0 = fmaf(x0, c, -x1 * s);
                float rot1 = fmaf(x0, s, x1 * c);
                x0 = rot0;
                x1 = rot1;
            }
            if (is_q) {
                uint16_t* qd = q_inout + ((size_t)r * Hq + lh) * D;
                qd[d0] = store16(x0, dtype);
                qd[d1] = store16(x1, dtype);
            } else {
                const uint16_t* vs = v_in + ((size_t)r * Hkv + lh) * D;
                if (g_kv_q4) { /* quantised below, from the un-rounded rotated key and from the value as given */
                    k_row[d0] = x0;
                    k_row[d1] = x1;
                    v_row[d0] = load16(vs[d0], dtype);
                    v_row[d1] = load16(vs[d1], dtype);
                } else {
                    cache_k[dst + d0] = store16(x0, dtype);
                    cache_k[dst + d1] = store16(x1, dtype);
                    cache_v[dst + d0] = vs[d0];
                    cache_v[dst + d1] = vs[d1];
                }
            }
        }
        if (!is_q && g_kv_q4) {
            ko_q4kv_quantize(k_row, D / KO_Q4_GROUP, (uint8_t*)cache_k + dst / KO_Q4_GROUP * KO_Q4_BLOCK_BYTES);
            ko_q4kv_quantize(v_row, D / KO_Q4_GROUP, (uint8_t*)cache_v + dst / KO_Q4_GROUP * KO_Q4_BLOCK_BYTES);
        }
    }
}

/* ---- decode stage 1: one work tile x one query head -------------------------- */

/* Per-lane element ownership of the shader: D=64 -> 2 consecutive elements per lane
 * (metal:280), D=128 -> 4 (metal:346), otherwise 8 with a d<D guard (metal:424). */
static inline uint32_t lane_width(uint32_t D) { return D == 64u ? 2u : (D == 128u ? 4u : 8u); }

typedef struct {
    float m, l;
    float o[256];
} ko_state;

/* AttentionMaskVariant::SlidingWindowCausal { window_size } (crates/kriya-core/src/descriptor.rs:63-70): the reference
 * declares the mask and no kernel reads it.  Semantics restated here: a query at position p attends the window_size most
 * recent positions, itself included, i.e. keys p + 1 - window_size ..= p.  0 = plain causal.  Every caller of
 * stream_blocks describes the keys visible to ONE query as a row whose last token is the query's own position, so the
 * window is the last `window` tokens of the row. */
static uint32_t g_attention_window = 0u;
KO_EXPORT void ko_set_attention_window(uint32_t window_size) { g_attention_window = window_size; }

/* The token-serial online softmax of metal:289-326 / 357-398 / 430-467 over logical
 * blocks [blk_begin, blk_end) of request `req`, in fp32, shader operation order. */
static void stream_blocks(const uint16_t* q_row, const uint16_t* cache_k, const uint16_t* cache_v,
                          const int32_t* indptr, const int32_t* indices, const int32_t* last_len,
                          uint32_t req, uint32_t kv_head, uint32_t blk_begin, uint32_t blk_end,
                          const ko_gqa_params* p, int dtype, ko_state* st) {
    const uint32_t D = p->head_dim, W = lane_width(D), page = p->block_size_tokens;
    const int32_t row0 = indptr[req], row1 = indptr[req + 1];
    const uint32_t total = (uint32_t)((row1 - row0) > 0 ? (row1 - row0) : 0);
    const int softcap = p->logit_softcap > 0.0f;
    float q[256];
    for (uint32_t d = 0; d < 256; ++d) q[d] = 0.0f;
    for (uint32_t d = 0; d < D; ++d) q[d] = load16(q_row[d], dtype) * p->sm_scale; /* metal:281,350,425 */
    st->m = -INFINITY;
    st->l = 0.0f;
    for (uint32_t d = 0; d < 256; ++d) st->o[d] = 0.0f;
    if (blk_end > total) blk_end = total; /* metal:274 */
    const size_t tok_stride = (size_t)p->num_kv_heads * D;
    uint32_t tok_first = 0u; /* first token inside the sliding window */
    if (g_attention_window != 0u && total > 0u) {
        int32_t ll = last_len[req];
        const uint32_t row_tokens = (total - 1u) * page + (uint32_t)(ll > 1 ? ll : 1);
        tok_first = row_tokens > g_attention_window ? row_tokens - g_attention_window : 0u;
    }
    for (uint32_t lb = blk_begin; lb < blk_end; ++lb) {
        const uint32_t phys = (uint32_t)indices[row0 + (int32_t)lb];
        uint32_t valid = page;
        if (lb + 1u == total) { /* metal:291-293 */
            int32_t ll = last_len[req];
            valid = (uint32_t)(ll > 1 ? ll : 1);
        }
        const size_t base = ((size_t)phys * page * p->num_kv_heads + kv_head) * D;
        for (uint32_t t = 0; t < valid; ++t) {
            if (lb * page + t < tok_first) continue;
            const size_t kr = base + t * tok_stride; /* element index of the token's K (and V) row */
            float lane[32];
            for (uint32_t l = 0; l < 32; ++l) {
                const uint32_t d0 = l * W;
                float dot;
                if (W == 2u) { /* metal:306 */
                    dot = fmaf(q[d0], kv_elem(cache_k, kr + d0, dtype), q[d0 + 1] * kv_elem(cache_k, kr + d0 + 1, dtype));
                } else if (W == 4u) { /* metal:375 */
                    dot = fmaf(q[d0], kv_elem(cache_k, kr + d0, dtype),
                               fmaf(q[d0 + 1], kv_elem(cache_k, kr + d0 + 1, dtype),
                                    fmaf(q[d0 + 2], kv_elem(cache_k, kr + d0 + 2, dtype),
                                         q[d0 + 3] * kv_elem(cache_k, kr + d0 + 3, dtype))));
                } else { /* metal:441-448 */
                    dot = 0.0f;
                    for (uint32_t i = 0; i < 8u; ++i)
                        if (d0 + i < D) dot = fmaf(q[d0 + i], kv_elem(cache_k, kr + d0 + i, dtype), dot);
                }
                lane[l] = dot;
            }
            float score = simd_sum32(lane);
            if (softcap) score = safe_tanh(score / p->logit_softcap) * p->logit_softcap; /* metal:308-310 */
            float m_new = fmaxf(st->m, score);
            float alpha = expf(clampf(st->m - m_new, -80.0f, 0.0f));
            float beta = expf(clampf(score - m_new, -80.0f, 0.0f));
            st->l = fmaf(st->l, alpha, beta);
            for (uint32_t d = 0; d < D; ++d) st->o[d] = fmaf(st->o[d], alpha, beta * kv_elem(cache_v, kr + d, dtype));
            st->m = m_new;
        }
    }
}

/* metal:242-495 for every (tile, query head).  Non-split tiles write `final_out` (16-bit);
 * split tiles write the normalised partial and lse = m + log(max(l,1e-12)) at slot
 * tile_split_idx[tile] (metal:332-342). */
KO_EXPORT void ko_decode_stage1(const uint16_t* q, const uint16_t* cache_k, const uint16_t* cache_v,
                                const int32_t* indptr, const int32_t* indices, const int32_t* last_len,
                                const ko_tile* tiles, uint32_t num_tiles, const uint32_t* tile_split_idx,
                                uint16_t* final_out, float* partial_out, float* partial_lse,
                                const ko_gqa_params* p, int dtype) {
    const uint32_t Hq = p->num_q_heads, D = p->head_dim, G = Hq / p->num_kv_heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t job = 0; job < (int64_t)num_tiles * Hq; ++job) {
        const uint32_t ti = (uint32_t)(job / Hq), qh = (uint32_t)(job % Hq);
        const ko_tile tile = tiles[ti];
        const uint32_t req = tile.request_idx;
        ko_state st;
        const size_t q_base = ((size_t)req * Hq + qh) * D;
        stream_blocks(q + q_base, cache_k, cache_v, indptr, indices, last_len, req, qh / G, tile.kv_block_start,
                      tile.kv_block_start + tile.kv_block_count, p, dtype, &st);
        const float inv_l = 1.0f / fmaxf(st.l, 1e-12f);
        if (tile.is_split_k == 0u) {
            for (uint32_t d = 0; d < D; ++d) final_out[q_base + d] = store16(st.o[d] * inv_l, dtype);
        } else {
            const size_t lse_idx = ((size_t)req * Hq + qh) * p->max_split_k_tiles + tile_split_idx[ti];
            for (uint32_t d = 0; d < D; ++d) partial_out[lse_idx * D + d] = st.o[d] * inv_l;
            partial_lse[lse_idx] = st.m + logf(fmaxf(st.l, 1e-12f));
        }
    }
}

/* metal:1474-1525: lse-weighted merge of the normalised partials of one request row. */
KO_EXPORT void ko_split_k_reduce(const float* partial_out, const float* partial_lse, const uint32_t* num_splits_req,
                                 uint16_t* final_out, uint32_t batch, const ko_gqa_params* p, int dtype) {
    const uint32_t Hq = p->num_q_heads, D = p->head_dim;
    for (uint32_t req = 0; req < batch; ++req) {
        const uint32_t ns = num_splits_req[req];
        if (ns <= 1u) continue; /* metal:1486-1488 */
        for (uint32_t qh = 0; qh < Hq; ++qh) {
            const size_t lse_base = ((size_t)req * Hq + qh) * p->max_split_k_tiles;
            float max_lse = -INFINITY;
            for (uint32_t s = 0; s < ns; ++s) max_lse = fmaxf(max_lse, partial_lse[lse_base + s]);
            float sum_exp = 0.0f;
            for (uint32_t s = 0; s < ns; ++s) sum_exp += expf(partial_lse[lse_base + s] - max_lse);
            const float inv_denom = 1.0f / fmaxf(sum_exp, 1e-12f);
            for (uint32_t d = 0; d < D; ++d) {
                float acc = 0.0f;
                for (uint32_t s = 0; s < ns; ++s) {
                    float w = expf(partial_lse[lse_base + s] - max_lse) * inv_denom;
                    acc = fmaf(w, partial_out[(lse_base + s) * D + d], acc);
                }
                final_out[((size_t)req * Hq + qh) * D + d] = store16(acc, dtype);
            }
        }
    }
}

/* Whole-row decode: each (request, query head) streams all of its blocks as one tile.
 * This is the "fp32 re-evaluation of the reference path" the CUDA decode kernel is held
 * to (it equals ko_decode_stage1 with one non-split tile per request).  out_f32, when
 * not NULL, receives the un-rounded result. */
KO_EXPORT void ko_decode(const uint16_t* q, const uint16_t* cache_k, const uint16_t* cache_v, const int32_t* indptr,
                         const int32_t* indices, const int32_t* last_len, uint32_t batch, uint16_t* out,
                         float* out_f32, const ko_gqa_params* p, int dtype) {
    const uint32_t Hq = p->num_q_heads, D = p->head_dim, G = Hq / p->num_kv_heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t job = 0; job < (int64_t)batch * Hq; ++job) {
        const uint32_t req = (uint32_t)(job / Hq), qh = (uint32_t)(job % Hq);
        ko_state st;
        const size_t q_base = ((size_t)req * Hq + qh) * D;
        const uint32_t nblk = (uint32_t)(indptr[req + 1] - indptr[req]);
        stream_blocks(q + q_base, cache_k, cache_v, indptr, indices, last_len, req, qh / G, 0u, nblk, p, dtype, &st);
        const float inv_l = 1.0f / fmaxf(st.l, 1e-12f);
        for (uint32_t d = 0; d < D; ++d) {
            if (out) out[q_base + d] = store16(st.o[d] * inv_l, dtype);
            if (out_f32) out_f32[q_base + d] = st.o[d] * inv_l;
        }
    }
}

/* Decode restricted to logical blocks [blk_begin[r], blk_end[r]) of every request, returning
 * the un-normalised state (m, l, o).  Used to check KV-axis sharding: ranks' states merged with
 * ko_merge_states must reproduce ko_decode. */
KO_EXPORT void ko_decode_partial(const uint16_t* q, const uint16_t* cache_k, const uint16_t* cache_v,
                                 const int32_t* indptr, const int32_t* indices, const int32_t* last_len,
                                 uint32_t batch, const uint32_t* blk_begin, const uint32_t* blk_end, float* out_m,
                                 float* out_l, float* out_o, const ko_gqa_params* p, int dtype) {
    const uint32_t Hq = p->num_q_heads, D = p->head_dim, G = Hq / p->num_kv_heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t job = 0; job < (int64_t)batch * Hq; ++job) {
        const uint32_t req = (uint32_t)(job / Hq), qh = (uint32_t)(job % Hq);
        ko_state st;
        const size_t row = (size_t)req * Hq + qh;
        stream_blocks(q + row * D, cache_k, cache_v, indptr, indices, last_len, req, qh / G, blk_begin[req],
                      blk_end[req], p, dtype, &st);
        out_m[row] = st.m;
        out_l[row] = st.l;
        for (uint32_t d = 0; d < D; ++d) out_o[row * D + d] = st.o[d];
    }
}

/* Merge `parts` un-normalised states per row: the a11 formula (metal:1493-1515) rewritten for
 * (m, l, o) instead of (lse, o/l): out = sum_s e^{m_s-M} o_s / sum_s e^{m_s-M} l_s. */
KO_EXPORT void ko_merge_states(const float* m, const float* l, const float* o, uint32_t parts, uint32_t rows,
                               uint32_t D, float* out_f32) {
    for (uint32_t r = 0; r < rows; ++r) {
        float M = -INFINITY;
        for (uint32_t s = 0; s < parts; ++s) M = fmaxf(M, m[(size_t)s * rows + r]);
        float den = 0.0f;
        for (uint32_t s = 0; s < parts; ++s) {
            float ms = m[(size_t)s * rows + r];
            if (ms > -INFINITY) den += expf(ms - M) * l[(size_t)s * rows + r];
        }
        const float inv = 1.0f / fmaxf(den, 1e-12f);
        for (uint32_t d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (uint32_t s = 0; s < parts; ++s) {
                float ms = m[(size_t)s * rows + r];
                if (ms > -INFINITY) acc = fmaf(expf(ms - M), o[((size_t)s * rows + r) * D + d], acc);
            }
            out_f32[(size_t)r * D + d] = acc * inv;
        }
    }
}

/* ---- speculative tree verification ------------------------------------------- */

typedef struct {
    uint32_t num_tree_nodes, num_q_heads, num_kv_heads, head_dim, block_size_tokens, prefix_kv_blocks, prefix_last_len;
    float sm_scale;
} ko_tree_params; /* TreeVerifyGqaParams, 32 bytes (enc:189-200, metal:1604-1613) */

/* One warp of bsr_paged_gqa_tree_verify (metal:1620-1729): lane l holds elements 4l..4l+3 (those below D), the score is
 * the butterfly sum of the lanes' fma chains, the recurrence uses plain exp (this kernel has no clamp), part A walks the
 * prefix pages of `page_indices`, part B the tree nodes the mask lets node i see.  The reference's own tests do not
 * cover this kernel: its parity is pinned by this restatement and by its agreement with the causal prefill when the
 * mask is lower-triangular (tests/test_oracle_numerics.py). */
KO_EXPORT void ko_tree_verify(const uint16_t* tree_q, const uint16_t* tree_k, const uint16_t* tree_v,
                              const uint16_t* cache_k, const uint16_t* cache_v, const int32_t* page_indices,
                              const uint8_t* tree_mask, uint16_t* tree_out, float* out_f32, const ko_tree_params* p,
                              int dtype) {
    const uint32_t N = p->num_tree_nodes, Hq = p->num_q_heads, Hkv = p->num_kv_heads, D = p->head_dim;
    const uint32_t G = Hq / Hkv, page = p->block_size_tokens;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t job = 0; job < (int64_t)N * Hq; ++job) {
        const uint32_t node = (uint32_t)(job / Hq), qh = (uint32_t)(job % Hq), kvh = qh / G;
        const size_t q_base = ((size_t)node * Hq + qh) * D;
        float q[128], o[128];
        for (uint32_t d = 0; d < 128; ++d) {
            q[d] = d < D ? load16(tree_q[q_base + d], dtype) * p->sm_scale : 0.0f; /* metal:1651-1654 */
            o[d] = 0.0f;
        }
        float m = -INFINITY, l = 0.0f;
        const uint32_t n_keys_prefix =
            p->prefix_kv_blocks ? (p->prefix_kv_blocks - 1u) * page + p->prefix_last_len : 0u; /* metal:1662-1664 */
        for (uint32_t key = 0; key < n_keys_prefix + N; ++key) {
            const uint16_t *kr, *vr;
            if (key < n_keys_prefix) { /* part A, metal:1660-1692 */
                const uint32_t phys = (uint32_t)page_indices[key / page];
                const size_t off = (((size_t)phys * page + key % page) * Hkv + kvh) * D;
                kr = cache_k + off;
                vr = cache_v + off;
            } else { /* part B, metal:1695-1718 */
                const uint32_t j = key - n_keys_prefix;
                if (tree_mask[(size_t)node * N + j] == 0) continue;
                const size_t off = ((size_t)j * Hkv + kvh) * D;
                kr = tree_k + off;
                vr = tree_v + off;
            }
            float lane[32];
            for (uint32_t ln = 0; ln < 32; ++ln) {
                float dot = 0.0f;
                for (uint32_t i = 0; i < 4u; ++i) {
                    const uint32_t d = ln * 4u + i;
                    if (d < D) dot = fmaf(q[d], load16(kr[d], dtype), dot);
                }
                lane[ln] = dot;
            }
            const float score = simd_sum32(lane);
            const float m_new = fmaxf(m, score);
            const float alpha = expf(m - m_new);
            const float beta = expf(score - m_new);
            l = fmaf(l, alpha, beta);
            for (uint32_t d = 0; d < D; ++d) o[d] = fmaf(o[d], alpha, beta * load16(vr[d], dtype));
            m = m_new;
        }
        const float inv_l = 1.0f / fmaxf(l, 1e-12f);
        for (uint32_t d = 0; d < D; ++d) {
            const float val = o[d] * inv_l;
            if (tree_out) tree_out[q_base + d] = store16(val, dtype);
            if (out_f32) out_f32[q_base + d] = val;
        }
    }
}

/* ---- causal prefill over the paged cache ------------------------------------- */

/* Query i of the chunk sits at absolute position prefix+i and attends cache positions
 * 0..=prefix+i of its sequence, token-serially with the decode recurrence
 * (metal:605-649 / 713-763).  The shader compares absolute key positions with the
 * chunk-relative query index (metal:606-609,1303-1306,1361), which is only right for
 * prefix 0; true causal masking is used here, which is what the reference's own CPU
 * check computes (tsc:1746-1775) and what its per-token plans describe
 * (crates/kriya-kv/src/bsr_paged.rs:631-644).  `table` holds the sequence's logical
 * blocks.  Scale is folded into q like the scalar kernels do (metal:570,679). */
KO_EXPORT void ko_prefill_causal(const uint16_t* q, const uint16_t* cache_k, const uint16_t* cache_v,
                                 const int32_t* table, uint32_t prefix_tokens, uint32_t num_tokens, uint16_t* out,
                                 float* out_f32, const ko_gqa_params* p, int dtype) {
    const uint32_t Hq = p->num_q_heads, D = p->head_dim, G = Hq / p->num_kv_heads, page = p->block_size_tokens;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t job = 0; job < (int64_t)num_tokens * Hq; ++job) {
        const uint32_t i = (uint32_t)(job / Hq), qh = (uint32_t)(job % Hq);
        const uint32_t visible = prefix_tokens + i + 1u;
        const uint32_t nblk = (visible + page - 1u) / page;
        int32_t indptr[2] = {0, (int32_t)nblk};
        int32_t last_len[1] = {(int32_t)(((prefix_tokens + i) % page) + 1u)}; /* bsr_paged.rs:642-644 */
        ko_state st;
        const size_t q_base = ((size_t)i * Hq + qh) * D;
        stream_blocks(q + q_base, cache_k, cache_v, indptr, table, last_len, 0u, qh / G, 0u, nblk, p, dtype, &st);
        const float inv_l = 1.0f / fmaxf(st.l, 1e-12f);
        for (uint32_t d = 0; d < D; ++d) {
            if (out) out[q_base + d] = store16(st.o[d] * inv_l, dtype);
            if (out_f32) out_f32[q_base + d] = st.o[d] * inv_l;
        }
    }
}

/* ---- copy-on-write block copy ------------------------------------------------- */

/* The reference emits (src,dst) pairs (bsr_paged.rs:412-420, collected at
 * crates/kriya-scheduler/src/orca_engine.rs:267-278) but ships no consumer.  Intended
 * semantics (docs/adr/0002-kv-cache-design.md:10): dst block := src block for every
 * layer, K and V.  Pairs are applied in order. */
KO_EXPORT void ko_block_copy(uint16_t* cache_k, uint16_t* cache_v, size_t layer_stride_elems, uint32_t num_layers,
                             size_t block_elems, const uint32_t* pairs, uint32_t num_pairs) {
    for (uint32_t i = 0; i < num_pairs; ++i) {
        const uint32_t src = pairs[2 * i], dst = pairs[2 * i + 1];
        for (uint32_t layer = 0; layer < num_layers; ++layer) {
            uint16_t* k = cache_k + layer * layer_stride_elems;
            uint16_t* v = cache_v + layer * layer_stride_elems;
            memmove(k + dst * block_elems, k + src * block_elems, block_elems * 2);
            memmove(v + dst * block_elems, v + src * block_elems, block_elems * 2);
        }
    }
}

/* Speculative-KV commit analogue (enc:3591-3664): row `node` of a staging buffer
 * [nodes, Hkv*D] is copied bitwise into (block, slot) of one layer's K and V. */
KO_EXPORT void ko_slot_write(uint16_t* cache_k, uint16_t* cache_v, const uint16_t* stage_k, const uint16_t* stage_v,
                             size_t kv_dim, uint32_t block_size, const uint32_t* triples, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t node = triples[3 * i], blk = triples[3 * i + 1], slot = triples[3 * i + 2];
        const size_t off = ((size_t)blk * block_size + slot) * kv_dim;
        memcpy(cache_k + off, stage_k + (size_t)node * kv_dim, kv_dim * 2);
        memcpy(cache_v + off, stage_v + (size_t)node * kv_dim, kv_dim * 2);
    }
}

/* ---- the reference's own CPU checks, restated -------------------------------- */

/* tsc:1182-1209: RoPE (rotate-half, transcendental) on un-rounded f32 inputs, then a plain
 * max/normalise softmax attention of the last token's q over `tokens` keys.  Hq=Hkv=1. */
KO_EXPORT void ko_ref_test_rope_softmax_attention(const float* q_raw, const float* k_raw, const float* v_raw,
                                                  uint32_t tokens, uint32_t D, float* expected) {
    float* keys = (float*)malloc(sizeof(float) * tokens * D);
    float* qrot = (float*)malloc(sizeof(float) * D);
    float* scores = (float*)malloc(sizeof(float) * tokens);
    for (uint32_t t = 0; t <= tokens; ++t) {
        const float* src = t < tokens ? k_raw + (size_t)t * D : q_raw + (size_t)(tokens - 1) * D;
        float* dst = t < tokens ? keys + (size_t)t * D : qrot;
        const uint32_t position = t < tokens ? t : tokens - 1;
        memcpy(dst, src, sizeof(float) * D);
        for (uint32_t i = 0; i < D / 2; ++i) {
            float exponent = -((float)(2 * i)) / (float)D;
            float angle = (float)position * powf(10000.0f, exponent);
            float s = sinf(angle), c = cosf(angle);
            dst[i] = src[i] * c - src[i + D / 2] * s;
            dst[i + D / 2] = src[i] * s + src[i + D / 2] * c;
        }
    }
    float max_score = -INFINITY;
    for (uint32_t t = 0; t < tokens; ++t) {
        float acc = 0.0f;
        for (uint32_t d = 0; d < D; ++d) acc += qrot[d] * keys[(size_t)t * D + d];
        scores[t] = acc / sqrtf((float)D);
        max_score = fmaxf(max_score, scores[t]);
    }
    float norm = 0.0f;
    for (uint32_t t = 0; t < tokens; ++t) norm += expf(scores[t] - max_score);
    for (uint32_t d = 0; d < D; ++d) {
        float acc = 0.0f;
        for (uint32_t t = 0; t < tokens; ++t) acc += (expf(scores[t] - max_score) / norm) * v_raw[(size_t)t * D + d];
        expected[d] = acc;
    }
    free(keys);
    free(qrot);
    free(scores);
}

/* tsc:1746-1775: causal softmax attention over one contiguous block of keys, on the
 * bf16-rounded inputs widened back to f32. */
KO_EXPORT void ko_ref_test_causal_prefill(const float* q, const float* k, const float* v, uint32_t num_tokens,
                                          uint32_t Hq, uint32_t Hkv, uint32_t D, float sm_scale, float* expected) {
    float* scores = (float*)malloc(sizeof(float) * num_tokens);
    for (uint32_t t = 0; t < num_tokens; ++t)
        for (uint32_t qh = 0; qh < Hq; ++qh) {
            const uint32_t kh = qh / (Hq / Hkv);
            const float* qv = q + ((size_t)t * Hq + qh) * D;
            float max_s = -INFINITY;
            for (uint32_t j = 0; j <= t; ++j) {
                const float* kv = k + ((size_t)j * Hkv + kh) * D;
                float dot = 0.0f;
                for (uint32_t d = 0; d < D; ++d) dot += qv[d] * kv[d];
                scores[j] = dot * sm_scale;
                max_s = fmaxf(max_s, scores[j]);
            }
            float sum_exp = 0.0f;
            for (uint32_t j = 0; j <= t; ++j) {
                scores[j] = expf(scores[j] - max_s);
                sum_exp += scores[j];
            }
            for (uint32_t d = 0; d < D; ++d) {
                float acc = 0.0f;
                for (uint32_t j = 0; j <= t; ++j) acc += (scores[j] / sum_exp) * v[((size_t)j * Hkv + kh) * D + d];
                expected[((size_t)t * Hq + qh) * D + d] = acc;
            }
        }
    free(scores);
}

/* rwv:327-362: online-softmax paged decode over `num_blocks` identity-mapped blocks, on the
 * UN-rounded f32 inputs (the test feeds q_f32/k_f32/v_f32 to its CPU loop). */
KO_EXPORT void ko_ref_test_online_decode(const float* q, const float* k, const float* v, uint32_t batch, uint32_t Hq,
                                         uint32_t Hkv, uint32_t D, uint32_t num_blocks, uint32_t block_sz,
                                         float* expected) {
    const float sm_scale = 1.0f / sqrtf((float)D);
    const uint32_t G = Hq / Hkv;
    float* acc = (float*)malloc(sizeof(float) * D);
    for (uint32_t b = 0; b < batch; ++b)
        for (uint32_t qh = 0; qh < Hq; ++qh) {
            const uint32_t kvh = qh / G;
            float m_i = -INFINITY, l_i = 0.0f;
            for (uint32_t d = 0; d < D; ++d) acc[d] = 0.0f;
            for (uint32_t blk = 0; blk < num_blocks; ++blk)
                for (uint32_t tok = 0; tok < block_sz; ++tok) {
                    const size_t off = (((size_t)blk * block_sz + tok) * Hkv + kvh) * D;
                    float score = 0.0f;
                    for (uint32_t d = 0; d < D; ++d) score += q[((size_t)b * Hq + qh) * D + d] * k[off + d];
                    score *= sm_scale;
                    float m_new = fmaxf(m_i, score);
                    float alpha = expf(m_i - m_new), beta = expf(score - m_new);
                    l_i = l_i * alpha + beta;
                    for (uint32_t d = 0; d < D; ++d) acc[d] = acc[d] * alpha + beta * v[off + d];
                    m_i = m_new;
                }
            const float inv_l = 1.0f / fmaxf(l_i, 1e-12f);
            for (uint32_t d = 0; d < D; ++d) expected[((size_t)b * Hq + qh) * D + d] = acc[d] * inv_l;
        }
    free(acc);
}

KO_EXPORT int ko_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
KO_EXPORT void ko_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
