// Part of the elixir_b200 CUDA library (C ABI: include/elixir_b200.h).  See elx_common.cuh for the
// overview of the kernels and of how the sources are divided.
#include "elx_common.cuh"

namespace elx {

thread_local char t_cuda_err[256] = "";

Tuning g_tune;

int g_sm_count[64];   // per device ordinal, 0 = not queried yet

int record_cuda(cudaError_t e) {
    if (e == cudaSuccess) return ELX_OK;
    snprintf(t_cuda_err, sizeof(t_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
    return ELX_ERR_LAUNCH;
}

// SM count of the current device, or a negative status.
int sm_count() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        record_cuda(e);
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    if (dev < 0 || dev >= 64) return ELX_ERR_NODEVICE;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || n <= 0) {
            record_cuda(e);
            (void)cudaGetLastError();
            return ELX_ERR_NODEVICE;
        }
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

int grid_for(int64_t work_items, int ctas_per_sm) {
    const int sms = sm_count();
    if (sms < 0) return sms;
    int64_t g = static_cast<int64_t>(sms) * ctas_per_sm;
    if (g > work_items) g = work_items;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}

int capped(int resident, int cap) { return cap > 0 && cap < resident ? cap : resident; }

}  // namespace elx

using namespace elx;

namespace {

// ------------------------------------------------------------------------------------------------
// control block
// ------------------------------------------------------------------------------------------------

__global__ void ctl_init_kernel(ElxCtl* ctl, float initial_scale) {
    uint32_t* w = reinterpret_cast<uint32_t*>(ctl);
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(ElxCtl) / 4); i += blockDim.x) w[i] = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
        ctl->scale = initial_scale;
        ctl->div_scale = -1.0f;
        ctl->clip_coef = 1.0f;
    }
}

__device__ __forceinline__ bool is_pow2_float(float x) {
    const uint32_t u = __float_as_uint(x);
    const uint32_t ex = (u >> 23) & 0xFFu;
    // normal, positive, zero mantissa, and the reciprocal is normal too
    return (u >> 31) == 0 && (u & 0x7FFFFFu) == 0 && ex >= 2 && ex <= 252;
}

// The three outcomes of the per-step decision (one thread).  `scale` is the loss scale on entry; the
// new scale is returned.

// a wait gave up earlier (a peer never arrived, a copy never completed): the gradients may be incomplete, so
// nothing is updated; the scaler is left alone because no overflow was observed
__device__ float decide_forced_skip(ElxCtl* ctl, float scale) {
    ctl->skip = 1;
    ctl->skipped_steps += 1;
    ctl->forced_skips += 1;
    ctl->div_scale = -1.0f;
    ctl->inv_div = 0.0f;
    return scale;
}

__device__ float decide_overflow(ElxCtl* ctl, const ElxScalerCfg& cfg, float scale) {
    ctl->skip = 1;
    ctl->skipped_steps += 1;
    ctl->div_scale = -1.0f;
    ctl->inv_div = 0.0f;
    if (cfg.dynamic) {
        ctl->hysteresis_step += 1;
        ctl->growth_step = 0;
        if (ctl->hysteresis_step >= cfg.hysteresis) {
            scale = scale * cfg.backoff_factor;
            if (cfg.min_scale > 0.0f) scale = fmaxf(scale, cfg.min_scale);
        }
    }
    return scale;
}

__device__ float decide_apply(ElxCtl* ctl, const ElxScalerCfg& cfg, const float* norm_sq, float scale) {
    ctl->skip = 0;
    // combined divisor from the scale as it was during backward
    double combined = static_cast<double>(scale);
    float clip_coef = 1.0f;
    if (cfg.max_norm > 0.0f && norm_sq != nullptr) {
        const double total_norm = sqrt(static_cast<double>(*norm_sq));
        const double clip = (total_norm / static_cast<double>(scale) + 1e-6) / static_cast<double>(cfg.max_norm);
        ctl->grad_norm = static_cast<float>(total_norm / static_cast<double>(scale));
        if (clip > 1.0) {
            combined = clip * static_cast<double>(scale);
            clip_coef = static_cast<float>(clip);
        }
    }
    ctl->clip_coef = clip_coef;
    float div = static_cast<float>(combined);
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
            if (cfg.max_scale > 0.0f) scale = fminf(scale, cfg.max_scale);
        }
    }
    return scale;
}

__global__ void step_begin_kernel(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq, uint32_t* chunk_flags,
                                  int n_chunk_flags) {
    // the per-chunk overflow words have been consumed through found_inf: clear them (all threads)
    for (int i = threadIdx.x; i < n_chunk_flags; i += blockDim.x) chunk_flags[i] = 0;
    if (threadIdx.x != 0) return;
    const bool found = ctl->found_inf != 0;
    float scale = ctl->scale;
    if (ctl->status & ELX_STAT_TIMEOUT) scale = decide_forced_skip(ctl, scale);
    else if (found) scale = decide_overflow(ctl, cfg, scale);
    else scale = decide_apply(ctl, cfg, norm_sq, scale);
    ctl->scale = scale;
    ctl->found_inf = 0;
}

// Single-pass step: the decision taken BEFORE the gradients have been looked at, on the assumption that they
// are clean; what it changes is saved so that elx_step_commit can take it back.
__global__ void step_begin_optimistic_kernel(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags) {
    for (int i = threadIdx.x; i < n_chunk_flags; i += blockDim.x) chunk_flags[i] = 0;
    if (threadIdx.x != 0) return;
    float scale = ctl->scale;
    ctl->repair = 0;
    if ((ctl->status & ELX_STAT_TIMEOUT) || ctl->found_inf != 0) {
        // known before the first update: decided for real, the kernels only refresh the working copies
        scale = (ctl->status & ELX_STAT_TIMEOUT) ? decide_forced_skip(ctl, scale) : decide_overflow(ctl, cfg, scale);
        ctl->spec_state = 2;
    } else {
        ctl->saved_scale = scale;
        ctl->saved_growth_step = ctl->growth_step;
        ctl->saved_hysteresis_step = ctl->hysteresis_step;
        ctl->saved_step = ctl->step;
        scale = decide_apply(ctl, cfg, nullptr, scale);
        ctl->spec_state = 1;
    }
    ctl->scale = scale;
    ctl->found_inf = 0;
}

__global__ void step_commit_kernel(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags) {
    for (int i = threadIdx.x; i < n_chunk_flags; i += blockDim.x) chunk_flags[i] = 0;
    if (threadIdx.x != 0) return;
    if (ctl->spec_state == 1) {
        const bool expired = (ctl->status & ELX_STAT_TIMEOUT) != 0;
        if (expired || ctl->found_inf != 0) {
            // the update that was written to the other set is not adopted: scaler state as before the optimistic
            // decision, then the decision an overflow (or an expired wait) calls for
            float scale = ctl->saved_scale;
            ctl->growth_step = ctl->saved_growth_step;
            ctl->hysteresis_step = ctl->saved_hysteresis_step;
            ctl->step = ctl->saved_step;
            scale = expired ? decide_forced_skip(ctl, scale) : decide_overflow(ctl, cfg, scale);
            ctl->scale = scale;
            ctl->repair = 1;
        } else {
            ctl->cur_set ^= 1u;
        }
    }
    // spec_state 2: decided up front, the working copies are already those of the untouched current set
    ctl->spec_state = 0;
    ctl->found_inf = 0;
}

}  // namespace

extern "C" {

int elx_version(void) { return ELX_ABI_VERSION; }

const char* elx_strerror(int status) {
    switch (status) {
        case ELX_OK: return "ok";
        case ELX_ERR_NULL: return "a required pointer is NULL";
        case ELX_ERR_ALIGN: return "a pointer is not aligned as required";
        case ELX_ERR_SIZE: return "a size or count is out of range";
        case ELX_ERR_DTYPE: return "unknown dtype code";
        case ELX_ERR_LAUNCH: return "CUDA launch failed";
        case ELX_ERR_ARG: return "inconsistent arguments";
        case ELX_ERR_NODEVICE: return "no usable CUDA device";
        case ELX_ERR_CAPACITY: return "request exceeds a fixed capacity";
    }
    return "unknown status";
}

const char* elx_last_cuda_error(void) { return t_cuda_err; }

int elx_set_tuning(const char* name, int value) {
    if (!name) return ELX_ERR_NULL;
    const Tuning def;
    struct Knob {
        const char* name;
        int* slot;
        int def;
        int lo, hi;
    };
    const Knob knobs[] = {
        {"adam_threads", &g_tune.adam_threads, def.adam_threads, 256, 512},
        {"adam_ctas_per_sm", &g_tune.adam_ctas_per_sm, def.adam_ctas_per_sm, 0, 32},
        {"probe_ctas_per_sm", &g_tune.probe_ctas_per_sm, def.probe_ctas_per_sm, 0, 32},
        {"probe_unroll", &g_tune.probe_unroll, def.probe_unroll, 4, 8},
        {"probe_variant", &g_tune.probe_variant, def.probe_variant, 0, 2},
        {"math_mode", &g_tune.math_mode, def.math_mode, 1, 2},
        {"adam_variant", &g_tune.adam_variant, def.adam_variant, 0, 1},
        {"pull_ctas_per_sm", &g_tune.pull_ctas_per_sm, def.pull_ctas_per_sm, 0, 32},
        {"pull_variant", &g_tune.pull_variant, def.pull_variant, 0, 1},
        {"adam_tma_ctas", &g_tune.adam_tma_ctas, def.adam_tma_ctas, 0, 1024},
        {"pull_tma_ctas", &g_tune.pull_tma_ctas, def.pull_tma_ctas, 0, 1024},
        {"adam_tma_stages", &g_tune.adam_tma_stages, def.adam_tma_stages, 0, 3},
    };
    for (const Knob& k : knobs) {
        if (strcmp(name, k.name) != 0) continue;
        if (value < 0) {
            *k.slot = k.def;
            return ELX_OK;
        }
        if (value < k.lo || value > k.hi) return ELX_ERR_ARG;
        if (k.slot == &g_tune.adam_threads && value != 256 && value != 512) return ELX_ERR_ARG;
        if (k.slot == &g_tune.probe_unroll && value != 4 && value != 8) return ELX_ERR_ARG;
        if (k.slot == &g_tune.adam_tma_stages && value != 0 && value != 3) return ELX_ERR_ARG;
        *k.slot = value;
        return ELX_OK;
    }
    return ELX_ERR_ARG;
}


int elx_ctl_init(ElxCtl* ctl, float initial_scale, void* stream) {
    if (!ctl) return ELX_ERR_NULL;
    if (!aligned(ctl, 16)) return ELX_ERR_ALIGN;
    if (!(initial_scale > 0.0f)) return ELX_ERR_ARG;
    ctl_init_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctl, initial_scale);
    return record_cuda(cudaGetLastError());
}

int elx_step_begin(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq, uint32_t* chunk_flags, int n_chunk_flags,
                   void* stream) {
    if (!ctl) return ELX_ERR_NULL;
    if (!aligned(ctl, 16) || (norm_sq && !aligned(norm_sq, 4)) || (chunk_flags && !aligned(chunk_flags, 4)))
        return ELX_ERR_ALIGN;
    if (n_chunk_flags < 0) return ELX_ERR_SIZE;
    if (!chunk_flags) n_chunk_flags = 0;
    if (cfg.dynamic) {
        if (!(cfg.growth_factor > 0.0f) || !(cfg.backoff_factor > 0.0f) || cfg.growth_interval <= 0 ||
            cfg.hysteresis < 0)
            return ELX_ERR_ARG;
    }
    if (cfg.max_norm > 0.0f && !norm_sq) return ELX_ERR_NULL;
    step_begin_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(ctl, cfg, norm_sq, chunk_flags, n_chunk_flags);
    return record_cuda(cudaGetLastError());
}

static int check_single_pass_args(ElxCtl* ctl, const ElxScalerCfg& cfg, uint32_t* chunk_flags, int* n_chunk_flags) {
    if (!ctl) return ELX_ERR_NULL;
    if (!aligned(ctl, 16) || (chunk_flags && !aligned(chunk_flags, 4))) return ELX_ERR_ALIGN;
    if (*n_chunk_flags < 0) return ELX_ERR_SIZE;
    if (!chunk_flags) *n_chunk_flags = 0;
    if (cfg.dynamic) {
        if (!(cfg.growth_factor > 0.0f) || !(cfg.backoff_factor > 0.0f) || cfg.growth_interval <= 0 ||
            cfg.hysteresis < 0)
            return ELX_ERR_ARG;
    }
    if (cfg.max_norm > 0.0f) return ELX_ERR_ARG;   // clipping needs the global norm before the first update
    return ELX_OK;
}

int elx_step_begin_optimistic(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags, void* stream) {
    const int rc = check_single_pass_args(ctl, cfg, chunk_flags, &n_chunk_flags);
    if (rc != ELX_OK) return rc;
    step_begin_optimistic_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(ctl, cfg, chunk_flags, n_chunk_flags);
    return record_cuda(cudaGetLastError());
}

int elx_step_commit(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags, void* stream) {
    const int rc = check_single_pass_args(ctl, cfg, chunk_flags, &n_chunk_flags);
    if (rc != ELX_OK) return rc;
    step_commit_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(ctl, cfg, chunk_flags, n_chunk_flags);
    return record_cuda(cudaGetLastError());
}

}  // extern "C"
