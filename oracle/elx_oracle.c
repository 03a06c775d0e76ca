/*
 * TEST INFRASTRUCTURE — CPU restatement of the chunk optimizer step.  Not part of the product:
 * only the test-suite, the smoke check and the CPU-baseline legs of the benchmark may load it.
 *
 * Parity status: the state machine (probe domain, skip, order of scale read / scaler update,
 * copy-back on skip, shard geometry) is pinned against hpcaitech/Elixir's own Python code run on
 * CPU (fixtures under tests/golden/).  The Adam arithmetic and the dynamic loss scaler live in
 * ColossalAI, which Elixir does not pin and which is not available offline: for those two the
 * oracle restates the published algorithm and is pinned against torch.optim.Adam / AdamW on CPU and,
 * for the scaler with hysteresis 1, against torch's own AMP scale update — "parity unpinned" with
 * respect to ColossalAI itself.
 *
 * What each function follows (paths inside hpcaitech/Elixir unless stated otherwise):
 *   orc_probe        elixir/chunk/core/chunk.py:214-216  set_overflow_flag (isinf|isnan, any)
 *                    over shard[:valid_end]               chunk.py:345-354
 *   orc_l2sq         chunk.py:218-221  set_l2_norm: float().norm(2) ** 2
 *   orc_cast         chunk.py:413-415  shard.copy_(fp32 shard): round to nearest even
 *   orc_step_begin   elixir/wrapper/optimizer.py:192-209 (found_inf -> skip; combined scale read
 *                    before the scaler update; sentinel -1 when it equals 1: :166-183) together
 *                    with ColossalAI DynamicGradScaler.update (overflow: hysteresis_step += 1,
 *                    growth_step = 0, backoff once hysteresis_step >= hysteresis, clamped to
 *                    min_scale; clean: growth_step += 1 and, at growth_interval, both counters
 *                    reset and scale grown, clamped to max_scale)
 *   orc_adam_f32     ColossalAI/Apex multi-tensor Adam functor as called with div_scale at
 *                    optimizer.py:216: g /= div; L2 mode g += wd*p; m = b1*m + (1-b1)*g;
 *                    v = b2*v + (1-b2)*g*g; update = (m/bc1) / (sqrt(v/bc2) + eps)
 *                    [+ wd*p decoupled]; p -= lr*update — strict fp32, this operation order
 *   orc_adam_f64     the same expression evaluated in double from the same fp32 inputs
 *   orc_reduce_avg   chunk.py:298-303  payload /= W (rounded in the chunk dtype), then SUM
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "elixir_b200.h"

/* ---- 16-bit float conversions, bit-exact, no compiler half types --------------------------- */

static inline float bits_f32(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint32_t f32_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

static float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t ex = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (ex == 0x1Fu) return bits_f32(sign | 0x7F800000u | (man << 13));
    if (ex == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: man * 2^-24 */
        float v = (float)man * (1.0f / 16777216.0f);
        return sign ? -v : v;
    }
    return bits_f32(sign | ((ex + 112u) << 23) | (man << 13));
}

static uint16_t f32_to_f16_rne(float f) {
    uint32_t x = f32_bits(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) {               /* inf / nan */
        if (ax > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((ax >> 13) & 0x3FFu));
        return (uint16_t)(sign | 0x7C00u);
    }
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);   /* >= 65520 rounds to inf */
    if (ax < 0x33000001u) return sign;                            /* <= 2^-25 rounds to zero */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t base;
    if (e < -14) {                          /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;   /* carries propagate into the exponent */
    return (uint16_t)(sign | (base + q));
}

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

static uint16_t f32_to_bf16_rne(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);   /* quiet nan */
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

static inline float lowp_get(const void* p, int dtype, int64_t i) {
    if (dtype == ELX_F16) return f16_to_f32(((const uint16_t*)p)[i]);
    if (dtype == ELX_BF16) return bf16_to_f32(((const uint16_t*)p)[i]);
    return ((const float*)p)[i];
}

static inline void lowp_set(void* p, int dtype, int64_t i, float v) {
    if (dtype == ELX_F16) ((uint16_t*)p)[i] = f32_to_f16_rne(v);
    else if (dtype == ELX_BF16) ((uint16_t*)p)[i] = f32_to_bf16_rne(v);
    else ((float*)p)[i] = v;
}

/* exported for the tests of the conversions themselves */
uint16_t orc_f32_to_f16(float f) { return f32_to_f16_rne(f); }
uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

/* ---- probe, norm, cast ---------------------------------------------------------------------- */

int orc_probe(const void* g, int dtype, int64_t n_valid) {
    int bad = 0;
    if (dtype == ELX_F32) {
        const uint32_t* u = (const uint32_t*)g;
#pragma omp parallel for reduction(| : bad)
        for (int64_t i = 0; i < n_valid; ++i) bad |= ((u[i] & 0x7F800000u) == 0x7F800000u);
    } else {
        const uint16_t mask = dtype == ELX_F16 ? 0x7C00u : 0x7F80u;
        const uint16_t* u = (const uint16_t*)g;
#pragma omp parallel for reduction(| : bad)
        for (int64_t i = 0; i < n_valid; ++i) bad |= ((u[i] & mask) == mask);
    }
    return bad;
}

double orc_l2sq(const void* g, int dtype, int64_t n_valid) {
    double s = 0.0;
#pragma omp parallel for reduction(+ : s)
    for (int64_t i = 0; i < n_valid; ++i) {
        double f = (double)lowp_get(g, dtype, i);
        s += f * f;
    }
    return s;
}

void orc_cast(const float* src, void* dst, int dtype, int64_t n) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) lowp_set(dst, dtype, i, src[i]);
}

/* Gradient averaging as the reference does it: every rank's value is divided by W and rounded in
 * the chunk dtype, then the W quotients are summed in rank order with a rounding after each add. */
void orc_reduce_avg(const void* const* ranks, int world, int dtype, int64_t n, void* out) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) {
        float acc = 0.0f;
        for (int r = 0; r < world; ++r) {
            float q = lowp_get(ranks[r], dtype, i) / (float)world;
            if (dtype == ELX_F16) q = f16_to_f32(f32_to_f16_rne(q));
            else if (dtype == ELX_BF16) q = bf16_to_f32(f32_to_bf16_rne(q));
            if (r == 0) acc = q;
            else {
                acc = acc + q;
                if (dtype == ELX_F16) acc = f16_to_f32(f32_to_f16_rne(acc));
                else if (dtype == ELX_BF16) acc = bf16_to_f32(f32_to_bf16_rne(acc));
            }
        }
        lowp_set(out, dtype, i, acc);
    }
}

/* The pull reduce-scatter of the NVLink path: sum over ranks, in rank order, of float(x_r) * (1/W) in
 * fp32, rounded once to the chunk dtype (elx_pull_reduce_multi). */
void orc_reduce_avg_f32acc(const void* const* ranks, int world, int dtype, int64_t n, void* out) {
    const float inv_w = 1.0f / (float)world;
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) {
        float acc = 0.0f;
        for (int r = 0; r < world; ++r) acc = fmaf(lowp_get(ranks[r], dtype, i), inv_w, acc);
        lowp_set(out, dtype, i, acc);
    }
}

/* ---- step decision + loss scaler (host copy of the control block) --------------------------- */

void orc_ctl_init(ElxCtl* ctl, float initial_scale) {
    memset(ctl, 0, sizeof(*ctl));
    ctl->scale = initial_scale;
    ctl->div_scale = -1.0f;
    ctl->clip_coef = 1.0f;
}

static int is_pow2_float(float x) {
    uint32_t u = f32_bits(x);
    uint32_t ex = (u >> 23) & 0xFFu;
    return (u >> 31) == 0 && (u & 0x7FFFFFu) == 0 && ex >= 2 && ex <= 252;
}

void orc_step_begin(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq) {
    int found = ctl->found_inf != 0;
    float scale = ctl->scale;
    if (found) {
        ctl->skip = 1;
        ctl->skipped_steps += 1;
        ctl->div_scale = -1.0f;
        ctl->inv_div = 0.0f;
        if (cfg.dynamic) {
            ctl->hysteresis_step += 1;
            ctl->growth_step = 0;
            if (ctl->hysteresis_step >= cfg.hysteresis) {
                scale = scale * cfg.backoff_factor;
                if (cfg.min_scale > 0.0f && scale < cfg.min_scale) scale = cfg.min_scale;
            }
        }
    } else {
        ctl->skip = 0;
        double combined = (double)scale;
        float clip_coef = 1.0f;
        if (cfg.max_norm > 0.0f && norm_sq) {
            double total_norm = sqrt((double)*norm_sq);
            double clip = (total_norm / (double)scale + 1e-6) / (double)cfg.max_norm;
            ctl->grad_norm = (float)(total_norm / (double)scale);
            if (clip > 1.0) {
                combined = clip * (double)scale;
                clip_coef = (float)clip;
            }
        }
        ctl->clip_coef = clip_coef;
        float div = (float)combined;
        if (combined == 1.0) div = -1.0f;
        ctl->div_scale = div;
        ctl->inv_div = (div > 0.0f && is_pow2_float(div)) ? 1.0f / div : 0.0f;
        ctl->step += 1;
        if (cfg.dynamic) {
            ctl->growth_step += 1;
            if (ctl->growth_step == cfg.growth_interval) {
                ctl->growth_step = 0;
                ctl->hysteresis_step = 0;
                scale = scale * cfg.growth_factor;
                if (cfg.max_scale > 0.0f && scale > cfg.max_scale) scale = cfg.max_scale;
            }
        }
    }
    ctl->scale = scale;
    ctl->found_inf = 0;
}

/* ---- Adam ------------------------------------------------------------------------------------- */

static void bias_corrections(const ElxHyper* h, int step, float* bc1, float* bc2) {
    *bc1 = 1.0f;
    *bc2 = 1.0f;
    if (h->bias_correction) {
        *bc1 = (float)(1.0 - pow((double)h->beta1, (double)step));
        *bc2 = (float)(1.0 - pow((double)h->beta2, (double)step));
    }
}

/* Strict fp32 (compile with -ffp-contract=off), reference operation order.  Updates p, m, v on
 * [begin, end); does not touch the low-precision array (the copy-back is orc_cast). */
void orc_adam_f32(float* p, float* m, float* v, const void* g, int dtype, int64_t begin, int64_t end,
                  ElxHyper h, int step, float div_scale) {
    float bc1, bc2;
    bias_corrections(&h, step, &bc1, &bc2);
    const float omb1 = 1.0f - h.beta1, omb2 = 1.0f - h.beta2;
#pragma omp parallel for
    for (int64_t i = begin; i < end; ++i) {
        float gi = lowp_get(g, dtype, i);
        if (div_scale > 0.0f) gi = gi / div_scale;
        float pi = p[i], mi = m[i], vi = v[i];
        if (!h.adamw_mode) gi = gi + h.weight_decay * pi;
        mi = h.beta1 * mi + omb1 * gi;
        vi = h.beta2 * vi + omb2 * gi * gi;
        float mhat = mi / bc1;
        float vhat = vi / bc2;
        float denom = sqrtf(vhat) + h.eps;
        float update = mhat / denom;
        if (h.adamw_mode) update = update + h.weight_decay * pi;
        pi = pi - h.lr * update;
        p[i] = pi;
        m[i] = mi;
        v[i] = vi;
    }
}

/* Double-precision evaluation of the same step from the same fp32 inputs; results rounded once to
 * fp32 on store.  The hyper-parameters enter as their fp32 values. */
void orc_adam_f64(float* p, float* m, float* v, const void* g, int dtype, int64_t begin, int64_t end,
                  ElxHyper h, int step, float div_scale) {
    double bc1 = 1.0, bc2 = 1.0;
    if (h.bias_correction) {
        bc1 = 1.0 - pow((double)h.beta1, (double)step);
        bc2 = 1.0 - pow((double)h.beta2, (double)step);
    }
    const double b1 = h.beta1, b2 = h.beta2, lr = h.lr, eps = h.eps, wd = h.weight_decay;
#pragma omp parallel for
    for (int64_t i = begin; i < end; ++i) {
        double gi = (double)lowp_get(g, dtype, i);
        if (div_scale > 0.0f) gi = gi / (double)div_scale;
        double pi = p[i], mi = m[i], vi = v[i];
        if (!h.adamw_mode) gi = gi + wd * pi;
        mi = b1 * mi + (1.0 - b1) * gi;
        vi = b2 * vi + (1.0 - b2) * gi * gi;
        double update = (mi / bc1) / (sqrt(vi / bc2) + eps);
        if (h.adamw_mode) update = update + wd * pi;
        pi = pi - lr * update;
        p[i] = (float)pi;
        m[i] = (float)mi;
        v[i] = (float)vi;
    }
}

/* One whole step over a chunk set, host memory, same tables as the device ABI: probe every chunk's
 * [0, n_valid), decide, update the segments (unless skipped), refresh every working copy over
 * [0, n_shard).  use_f64 selects the arithmetic of the update.  Returns the skip decision. */
int orc_step(const ElxChunkDesc* descs, int n_chunks, const ElxSeg* segs, const ElxHyper* hyper, int n_groups,
             ElxCtl* ctl, ElxScalerCfg cfg, int probe, int use_f64) {
    if (probe) {
        for (int c = 0; c < n_chunks; ++c)
            if (orc_probe(descs[c].grad_param, descs[c].dtype, descs[c].n_valid)) ctl->found_inf = 1;
    }
    float norm_sq = 0.0f;
    if (cfg.max_norm > 0.0f) {
        double s = 0.0;
        for (int c = 0; c < n_chunks; ++c) s += orc_l2sq(descs[c].grad_param, descs[c].dtype, descs[c].n_valid);
        norm_sq = (float)s;
    }
    orc_step_begin(ctl, cfg, cfg.max_norm > 0.0f ? &norm_sq : 0);
    for (int c = 0; c < n_chunks; ++c) {
        const ElxChunkDesc* d = &descs[c];
        if (!ctl->skip) {
            for (int s = d->seg_first; s < d->seg_first + d->seg_count; ++s) {
                if (segs[s].group < 0 || segs[s].group >= n_groups) continue;
                if (use_f64)
                    orc_adam_f64(d->master, d->exp_avg, d->exp_avg_sq, d->grad_param, d->dtype, segs[s].begin,
                                 segs[s].end, hyper[segs[s].group], ctl->step, ctl->div_scale);
                else
                    orc_adam_f32(d->master, d->exp_avg, d->exp_avg_sq, d->grad_param, d->dtype, segs[s].begin,
                                 segs[s].end, hyper[segs[s].group], ctl->step, ctl->div_scale);
            }
        }
        orc_cast(d->master, d->grad_param, d->dtype, d->n_shard);
    }
    return (int)ctl->skip;
}

int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}
