/*
 * CPU oracle for the paged-decode hot path.  TEST INFRASTRUCTURE ONLY: it is the checker the
 * CUDA kernels are compared with and the timed CPU baseline; the product never calls it.
 *
 * It restates, in plain C, the arithmetic of the reference's own CPU golden:
 *   - paged attention: tests/apitest/kernelstest/mix/test_paged_attention_common.py
 *       group_mm_torch :85-118, softmax_numpy :133-140, ref_masked_attention :229-276,
 *       ref_single_query_cached_kv_attention :278-366
 *   - MLA combined cache (V = first mlaVHeadSize columns of the K row):
 *       tests/apitest/opstest/python/operations/paged_attention/test_paged_attention_operation_mla.py
 *       ref_masked_attention :130-160, ref_single_query_cached_kv_attention :162-227
 *   - reshape_and_cache: tests/apitest/kernelstest/mix/test_reshape_and_cache.py :45-68
 *
 * Parity is pinned: tests/golden/ holds outputs of those reference Python functions on seeded
 * inputs, and tests/test_oracle_golden.py checks this file against them.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORACLE_FP16 = 0, ORACLE_BF16 = 1, ORACLE_INT8 = 2 };

static float g_half_lut[65536];
static int g_half_lut_ready = 0;

static float half_bits_to_float_slow(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static void ensure_lut(void)
{
    if (g_half_lut_ready) {
        return;
    }
    for (uint32_t i = 0; i < 65536; ++i) {
        g_half_lut[i] = half_bits_to_float_slow((uint16_t)i);
    }
    g_half_lut_ready = 1;
}

static inline float bf16_bits_to_float(uint16_t b)
{
    uint32_t bits = (uint32_t)b << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even, the rounding torch uses for .to(torch.bfloat16) */
static inline uint16_t float_to_bf16_bits(float f)
{
    uint32_t bits;
    memcpy(&bits, &f, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((bits >> 16) | 0x40u);
    }
    uint32_t lsb = (bits >> 16) & 1u;
    bits += 0x7fffu + lsb;
    return (uint16_t)(bits >> 16);
}

/* round-to-nearest-even float -> IEEE half */
static inline uint16_t float_to_half_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) {
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or == 2^-25, ties to even 0) */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (exp < -14) {
        shift = 13 + (-14 - exp);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) {
        q++;
    }
    return (uint16_t)(sign | (base + q));
}

static inline float load_elem(const void *p, int64_t idx, int dtype)
{
    if (dtype == ORACLE_FP16) {
        return g_half_lut[((const uint16_t *)p)[idx]];
    }
    if (dtype == ORACLE_BF16) {
        return bf16_bits_to_float(((const uint16_t *)p)[idx]);
    }
    return (float)((const int8_t *)p)[idx];
}

static inline float round_to_dtype(float v, int dtype)
{
    if (dtype == ORACLE_FP16) {
        return g_half_lut[float_to_half_bits(v)];
    }
    return bf16_bits_to_float(float_to_bf16_bits(v));
}

static inline void store_elem(void *p, int64_t idx, int dtype, float v)
{
    if (dtype == ORACLE_FP16) {
        ((uint16_t *)p)[idx] = float_to_half_bits(v);
    } else {
        ((uint16_t *)p)[idx] = float_to_bf16_bits(v);
    }
}

/*
 * Decode attention over a block-paged cache, one query token per sequence.
 *
 *  q            [batch, num_heads, dk]            q_dtype (fp16 | bf16)
 *  k_cache      [num_blocks, block_size, kv_heads, dk]      kv_dtype (fp16 | bf16 | int8)
 *  v_cache      [num_blocks, block_size, kv_heads, dv_row]  first dv columns are V
 *               (MLA combined cache: v_cache == k_cache, dv_row == dk, dv == mlaVHeadSize)
 *  block_tables [batch, max_blocks] int32;  context_lens [batch] int32
 *  k_descale/v_descale [kv_heads*dk]/[kv_heads*dv] fp32, k_offset/v_offset int32 (int8 cache only,
 *               any of them may be NULL): dequant = (float(x) + offset) * scale, all fp32
 *  out          [batch, num_heads, dv] q_dtype; out_high (nullable) same shape, fp32, with the
 *               un-rounded probabilities (the golden's "true_out")
 *
 *  mask         (nullable) fp32 additive bias, score(b, h, t) += mask[b*mask_batch_stride + h*mask_head_stride + t]:
 *               the alibi mask [batch, heads, 1, max_ctx] (strides heads*max_ctx, max_ctx), the plain
 *               mask [batch, 1, max_ctx] (strides max_ctx, 0) or one row for all (strides 0, 0)
 *  logn         (nullable) [batch] fp32, multiplies the scale of sequence b (SCALE_TYPE_LOGN)
 *
 * Follows ref_masked_attention: fp32 QK^T, * scale, + mask, fp32 softmax (max, exp, sum, divide),
 * P rounded to the query dtype, fp32 PV, result rounded to the query dtype.
 * A sequence with context_len == 0 is skipped and its output rows are left untouched.
 * Returns 0, or -1 on a bad argument.
 */
int oracle_paged_attention_ex(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_tables,
                              const int32_t *context_lens, const float *k_descale, const float *v_descale,
                              const int32_t *k_offset, const int32_t *v_offset, void *out, float *out_high,
                              int32_t batch, int32_t num_heads, int32_t kv_heads, int32_t dk, int32_t dv,
                              int32_t dv_row, int32_t block_size, int32_t max_blocks, int32_t q_dtype,
                              int32_t kv_dtype, float scale, int32_t nthreads, const float *mask,
                              int64_t mask_batch_stride, int64_t mask_head_stride, const float *logn)
{
    if (!q || !k_cache || !v_cache || !block_tables || !context_lens || !out || batch < 0 || num_heads <= 0 ||
        kv_heads <= 0 || num_heads % kv_heads != 0 || dk <= 0 || dv <= 0 || dv > dv_row || block_size <= 0) {
        return -1;
    }
    ensure_lut();
    const int group = num_heads / kv_heads;
#ifdef _OPENMP
    if (nthreads > 0) {
        omp_set_num_threads(nthreads);
    }
#else
    (void)nthreads;
#endif
    int64_t n_pairs = (int64_t)batch * kv_heads;
#pragma omp parallel
    {
        float *kf = NULL, *vf = NULL, *s = NULL, *p = NULL, *ph = NULL;
        int64_t cap = 0;
#pragma omp for schedule(dynamic, 1)
        for (int64_t pair = 0; pair < n_pairs; ++pair) {
            int b = (int)(pair / kv_heads);
            int hk = (int)(pair % kv_heads);
            int ctx = context_lens[b];
            if (ctx <= 0) {
                continue;
            }
            if (ctx > cap) {
                free(kf);
                free(vf);
                free(s);
                free(p);
                free(ph);
                cap = ctx;
                kf = (float *)malloc(sizeof(float) * (size_t)cap * dk);
                vf = (float *)malloc(sizeof(float) * (size_t)cap * dv);
                s = (float *)malloc(sizeof(float) * (size_t)cap);
                p = (float *)malloc(sizeof(float) * (size_t)cap);
                ph = (float *)malloc(sizeof(float) * (size_t)cap);
            }
            /* gather + dequantise this kv head's rows, as the golden does before the matmuls */
            for (int t = 0; t < ctx; ++t) {
                int64_t blk = block_tables[(int64_t)b * max_blocks + t / block_size];
                int64_t row = blk * block_size + t % block_size;
                int64_t kbase = (row * kv_heads + hk) * dk;
                int64_t vbase = (row * kv_heads + hk) * dv_row;
                float *kd = kf + (int64_t)t * dk;
                float *vd = vf + (int64_t)t * dv;
                for (int d = 0; d < dk; ++d) {
                    float x = load_elem(k_cache, kbase + d, kv_dtype);
                    if (kv_dtype == ORACLE_INT8) {
                        if (k_offset) {
                            x += (float)k_offset[hk * dk + d];
                        }
                        if (k_descale) {
                            x *= k_descale[hk * dk + d];
                        }
                    }
                    kd[d] = x;
                }
                for (int d = 0; d < dv; ++d) {
                    float x = load_elem(v_cache, vbase + d, kv_dtype);
                    if (kv_dtype == ORACLE_INT8) {
                        if (v_offset) {
                            x += (float)v_offset[hk * dv + d];
                        }
                        if (v_descale) {
                            x *= v_descale[hk * dv + d];
                        }
                    }
                    vd[d] = x;
                }
            }
            for (int g = 0; g < group; ++g) {
                int h = hk * group + g;
                float qf[1024];
                for (int d = 0; d < dk; ++d) {
                    qf[d] = load_elem(q, ((int64_t)b * num_heads + h) * dk + d, q_dtype);
                }
                float m = -INFINITY;
                for (int t = 0; t < ctx; ++t) {
                    const float *kd = kf + (int64_t)t * dk;
                    float acc = 0.f;
                    for (int d = 0; d < dk; ++d) {
                        acc += qf[d] * kd[d];
                    }
                    /* scale (times the sequence's logN factor), then the additive mask:
                     * test_paged_attention_common.py:252-254 and :345-347 of the reference */
                    acc *= logn ? scale * logn[b] : scale;
                    if (mask) {
                        acc += mask[(int64_t)b * mask_batch_stride + (int64_t)h * mask_head_stride + t];
                    }
                    s[t] = acc;
                    if (acc > m) {
                        m = acc;
                    }
                }
                float sum = 0.f;
                for (int t = 0; t < ctx; ++t) {
                    float e = expf(s[t] - m);
                    s[t] = e;
                    sum += e;
                }
                for (int t = 0; t < ctx; ++t) {
                    float pr = s[t] / sum;
                    ph[t] = pr;
                    p[t] = round_to_dtype(pr, q_dtype);
                }
                int64_t obase = ((int64_t)b * num_heads + h) * dv;
                float acc_o[1024];
                float acc_h[1024];
                for (int d = 0; d < dv; ++d) {
                    acc_o[d] = 0.f;
                    acc_h[d] = 0.f;
                }
                for (int t = 0; t < ctx; ++t) {
                    const float *vd = vf + (int64_t)t * dv;
                    float pt = p[t], pht = ph[t];
                    for (int d = 0; d < dv; ++d) {
                        acc_o[d] += pt * vd[d];
                        acc_h[d] += pht * vd[d];
                    }
                }
                for (int d = 0; d < dv; ++d) {
                    store_elem(out, obase + d, q_dtype, acc_o[d]);
                    if (out_high) {
                        out_high[obase + d] = acc_h[d];
                    }
                }
            }
        }
        free(kf);
        free(vf);
        free(s);
        free(p);
        free(ph);
    }
    return 0;
}

int oracle_paged_attention(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_tables,
                           const int32_t *context_lens, const float *k_descale, const float *v_descale,
                           const int32_t *k_offset, const int32_t *v_offset, void *out, float *out_high,
                           int32_t batch, int32_t num_heads, int32_t kv_heads, int32_t dk, int32_t dv,
                           int32_t dv_row, int32_t block_size, int32_t max_blocks, int32_t q_dtype,
                           int32_t kv_dtype, float scale, int32_t nthreads)
{
    return oracle_paged_attention_ex(q, k_cache, v_cache, block_tables, context_lens, k_descale, v_descale, k_offset,
                                     v_offset, out, out_high, batch, num_heads, kv_heads, dk, dv, dv_row, block_size,
                                     max_blocks, q_dtype, kv_dtype, scale, nthreads, NULL, 0, 0, NULL);
}

/*
 * ReshapeAndCache: for each token i with slot = slot_mapping[i] >= 0 copy the token's
 * [num_heads * head_size] row into cache row `slot` (slot = block * block_size + offset);
 * negative slots are skipped (test_reshape_and_cache.py :56-64).  Pure byte copy.
 * Either (key,key_cache) or (value,value_cache) may be NULL (the K-only "SISO" variant).
 */
int oracle_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                             const int32_t *slot_mapping, int32_t num_tokens, int64_t k_row_bytes,
                             int64_t v_row_bytes, int64_t num_slots)
{
    if (!slot_mapping || num_tokens < 0) {
        return -1;
    }
    for (int i = 0; i < num_tokens; ++i) {
        int64_t slot = slot_mapping[i];
        if (slot < 0) {
            continue;
        }
        if (slot >= num_slots) {
            return -1;
        }
        if (key && key_cache) {
            memcpy((char *)key_cache + slot * k_row_bytes, (const char *)key + (int64_t)i * k_row_bytes,
                   (size_t)k_row_bytes);
        }
        if (value && value_cache) {
            memcpy((char *)value_cache + slot * v_row_bytes, (const char *)value + (int64_t)i * v_row_bytes,
                   (size_t)v_row_bytes);
        }
    }
    return 0;
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Decode attention with int8 Q, K, V (quantType TYPE_QUANT_QKV_ONLINE / OFFLINE): restates
 * tests/apitest/kernelstest/mix/test_paged_attention_common.py of the reference:
 *   group_mm_torch :104-110 (int32 matmuls, then * de_scale[head]), softmax_quant_numpy :142-166 (running
 *   maximum per tile, P quantised to int8 per tile: online with the tile's own maximum / 127, offline with
 *   the per-head pScale; both round through fp16 first), softmax_quant_numpy_online :169-227 (tiles of
 *   `tile_tokens` = its block_size_calc inside splits of `split_tokens` = its kv_split_per_core, the
 *   splits merged by their log-sum-exp), ref_masked_attention :256-265.
 * k_descale, v_descale, p_scale: [H] fp32 (p_scale NULL = online).  Output in `out_dtype`.
 * The result depends (slightly) on where the tiles fall, so the tile and split sizes are arguments.
 */
int oracle_paged_attention_qkv_quant(const int8_t *q, const int8_t *k_cache, const int8_t *v_cache,
                                     const int32_t *block_tables, const int32_t *context_lens, const float *k_descale,
                                     const float *v_descale, const float *p_scale, void *out, int32_t B, int32_t H,
                                     int32_t Hkv, int32_t D, int32_t block_size, int32_t max_blocks, int32_t out_dtype,
                                     float scale, int32_t tile_tokens, int32_t split_tokens, int32_t nthreads)
{
    if (B < 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || block_size <= 0 || tile_tokens <= 0 ||
        split_tokens <= 0 || (out_dtype != ORACLE_FP16 && out_dtype != ORACLE_BF16)) {
        return 1;
    }
    ensure_lut();
#ifdef _OPENMP
    if (nthreads > 0) {
        omp_set_num_threads(nthreads);
    }
#else
    (void)nthreads;
#endif
    const int group = H / Hkv;
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            const int len = context_lens[b];
            if (len <= 0) {
                continue;
            }
            const int hk = h / group;
            const int n_split = (int)(((int64_t)len + split_tokens - 1) / split_tokens);
            float *sim = (float *)malloc(sizeof(float) * (size_t)tile_tokens);
            int8_t *pq = (int8_t *)malloc((size_t)tile_tokens);
            int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)D);
            float *go = (float *)malloc(sizeof(float) * (size_t)D);
            float *po = (float *)malloc(sizeof(float) * (size_t)D * (size_t)n_split);
            float *pl = (float *)malloc(sizeof(float) * (size_t)n_split);
            if (!sim || !pq || !acc || !go || !po || !pl) {
                failed = 1;
                free(sim); free(pq); free(acc); free(go); free(po); free(pl);
                continue;
            }
            const int8_t *qrow = q + ((int64_t)b * H + h) * D;
            for (int si = 0; si < n_split; ++si) {
                const int s_begin = si * split_tokens;
                const int s_end = len < s_begin + split_tokens ? len : s_begin + split_tokens;
                float gm = -3.4028234663852886e38f, gl = 0.f;
                for (int t0 = s_begin, first = 1; t0 < s_end; t0 += tile_tokens, first = 0) {
                    const int n = s_end - t0 < tile_tokens ? s_end - t0 : tile_tokens;
                    float lm = -INFINITY;
                    for (int t = 0; t < n; ++t) {
                        const int tok = t0 + t;
                        const int blk = block_tables[(int64_t)b * max_blocks + tok / block_size];
                        const int8_t *krow = k_cache + (((int64_t)blk * block_size + tok % block_size) * Hkv + hk) * D;
                        int32_t dot = 0;
                        for (int d = 0; d < D; ++d) {
                            dot += (int32_t)qrow[d] * (int32_t)krow[d];
                        }
                        const float s = ((float)dot * k_descale[h]) * scale;
                        sim[t] = s;
                        lm = s > lm ? s : lm;
                    }
                    float hm, dm;
                    if (first) {
                        hm = lm;
                        dm = 0.f;
                    } else {
                        hm = gm > lm ? gm : lm;
                        dm = gm - hm;
                    }
                    gm = hm;
                    float row_sum = 0.f, row_maxp = 0.f;
                    for (int t = 0; t < n; ++t) {
                        sim[t] = expf(sim[t] - hm);
                        row_sum += sim[t];
                        row_maxp = sim[t] > row_maxp ? sim[t] : row_maxp;
                    }
                    float dsv;
                    if (p_scale == NULL) {
                        const float sc = row_maxp / 127.0f;
                        for (int t = 0; t < n; ++t) {
                            const float v16 = g_half_lut[float_to_half_bits(sim[t] / sc)];
                            pq[t] = (int8_t)rintf(v16);
                        }
                        dsv = v_descale[h] * row_maxp / 127.f;
                    } else {
                        for (int t = 0; t < n; ++t) {
                            const float v16 = g_half_lut[float_to_half_bits(sim[t] * p_scale[h])];
                            pq[t] = (int8_t)rintf(v16);
                        }
                        dsv = v_descale[h];
                    }
                    memset(acc, 0, sizeof(int32_t) * (size_t)D);
                    for (int t = 0; t < n; ++t) {
                        const int tok = t0 + t;
                        const int blk = block_tables[(int64_t)b * max_blocks + tok / block_size];
                        const int8_t *vrow = v_cache + (((int64_t)blk * block_size + tok % block_size) * Hkv + hk) * D;
                        const int32_t p = pq[t];
                        for (int d = 0; d < D; ++d) {
                            acc[d] += p * (int32_t)vrow[d];
                        }
                    }
                    if (first) {
                        gl = row_sum;
                        for (int d = 0; d < D; ++d) {
                            go[d] = (float)acc[d] * dsv;
                        }
                    } else {
                        const float e = expf(dm);
                        gl = gl * e + row_sum;
                        for (int d = 0; d < D; ++d) {
                            go[d] = go[d] * e + (float)acc[d] * dsv;
                        }
                    }
                }
                for (int d = 0; d < D; ++d) {
                    po[(size_t)si * D + d] = go[d] / gl;
                }
                pl[si] = logf(gl) + gm;
            }
            if (n_split > 1) {
                float lmax = -INFINITY, lsum = 0.f;
                for (int si = 0; si < n_split; ++si) {
                    lmax = pl[si] > lmax ? pl[si] : lmax;
                }
                for (int si = 0; si < n_split; ++si) {
                    lsum += expf(pl[si] - lmax);
                }
                const float logsum = logf(lsum) + lmax;
                for (int d = 0; d < D; ++d) {
                    go[d] = 0.f;
                }
                for (int si = 0; si < n_split; ++si) {
                    const float w = expf(pl[si] - logsum);
                    for (int d = 0; d < D; ++d) {
                        go[d] += po[(size_t)si * D + d] * w;
                    }
                }
            } else {
                memcpy(go, po, sizeof(float) * (size_t)D);
            }
            uint16_t *orow = (uint16_t *)out + ((int64_t)b * H + h) * D;
            for (int d = 0; d < D; ++d) {
                orow[d] = out_dtype == ORACLE_BF16 ? float_to_bf16_bits(go[d]) : float_to_half_bits(go[d]);
            }
            free(sim); free(pq); free(acc); free(go); free(po); free(pl);
        }
    }
    return failed;
}
