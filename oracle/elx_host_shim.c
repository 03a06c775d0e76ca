/*
 * TEST INFRASTRUCTURE — the elx_* C ABI implemented on HOST memory with the CPU oracle.
 *
 * The test-suite loads this in place of libelixir_b200.so (tests/_dist_workers.py) to run the host-side
 * logic of the package — chunk geometry, collectives over gloo, the ElixirOptimizer state machine —
 * on machines without a GPU.  The product never loads it.  Pointers are host pointers, the stream
 * argument is ignored, every call completes before it returns.  Arithmetic: elx_oracle.c (double
 * precision evaluation of the update, rounded to fp32).
 */
#include <stdint.h>
#include <string.h>

#include "elixir_b200.h"

int orc_probe(const void* g, int dtype, int64_t n_valid);
double orc_l2sq(const void* g, int dtype, int64_t n_valid);
void orc_cast(const float* src, void* dst, int dtype, int64_t n);
void orc_ctl_init(ElxCtl* ctl, float initial_scale);
void orc_step_begin(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq);
void orc_adam_f64(float* p, float* m, float* v, const void* g, int dtype, int64_t begin, int64_t end, ElxHyper h,
                  int step, float div_scale);

static int dtype_ok(int dt) { return dt == ELX_F16 || dt == ELX_BF16 || dt == ELX_F32; }
static int dtype_bytes(int dt) { return dt == ELX_F32 ? 4 : 2; }

int elx_version(void) { return ELX_ABI_VERSION; }
const char* elx_strerror(int status) { return status == ELX_OK ? "ok" : "host shim: argument rejected"; }
const char* elx_last_cuda_error(void) { return ""; }
int elx_set_tuning(const char* name, int value) {
    (void)value;
    return name ? ELX_OK : ELX_ERR_NULL;
}
int64_t elx_probe_scratch_elems(int64_t n_tiles) { return n_tiles < 0 ? 0 : n_tiles; }
int64_t elx_grad_check_static_max_elems(void) { return (int64_t)16384 * ELX_TILE; }

int elx_ctl_init(ElxCtl* ctl, float initial_scale, void* stream) {
    (void)stream;
    if (!ctl) return ELX_ERR_NULL;
    orc_ctl_init(ctl, initial_scale);
    return ELX_OK;
}

int elx_step_begin(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq, uint32_t* chunk_flags, int n_chunk_flags,
                   void* stream) {
    (void)stream;
    if (!ctl) return ELX_ERR_NULL;
    if (cfg.max_norm > 0.0f && !norm_sq) return ELX_ERR_NULL;
    if (n_chunk_flags < 0) return ELX_ERR_SIZE;
    if (ctl->status & ELX_STAT_TIMEOUT) {
        /* a wait gave up earlier: skip without touching the loss scaler (no reference counterpart) */
        ctl->skip = 1;
        ctl->skipped_steps += 1;
        ctl->forced_skips += 1;
        ctl->div_scale = -1.0f;
        ctl->inv_div = 0.0f;
        ctl->found_inf = 0;
    } else {
        orc_step_begin(ctl, cfg, norm_sq);
    }
    for (int i = 0; chunk_flags && i < n_chunk_flags; ++i) chunk_flags[i] = 0;
    return ELX_OK;
}

static const void* grad_of(const ElxChunkDesc* d) { return d->grad_src ? d->grad_src : d->grad_param; }

static int probe_common(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl, float* l2sq) {
    if (!g) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (n_valid < 0) return ELX_ERR_SIZE;
    if (orc_probe(g, dtype, n_valid)) {
        if (flag) *flag = 1;
        if (ctl) ctl->found_inf = 1;
    }
    if (l2sq) *l2sq = (float)orc_l2sq(g, dtype, n_valid);
    return ELX_OK;
}

int elx_grad_check(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl, float* l2sq, float* scratch,
                   int64_t scratch_elems, void* stream) {
    (void)scratch;
    (void)scratch_elems;
    (void)stream;
    return probe_common(g, dtype, n_valid, flag, ctl, l2sq);
}

int elx_grad_check_static(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl, float* l2sq,
                          void* stream) {
    (void)stream;
    if (l2sq && g && dtype_ok(dtype) && n_valid > elx_grad_check_static_max_elems()) return ELX_ERR_CAPACITY;
    return probe_common(g, dtype, n_valid, flag, ctl, l2sq);
}

int elx_reduce_epilogue(const void* src, void* dst, int dtype, int64_t n_shard, int64_t n_valid, uint32_t* flag,
                        ElxCtl* ctl, float* l2sq, float* scratch, int64_t scratch_elems, void* stream) {
    (void)scratch;
    (void)scratch_elems;
    (void)stream;
    if (!src || !dst) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (n_shard < 0 || n_valid < 0 || n_valid > n_shard) return ELX_ERR_SIZE;
    memmove(dst, src, (size_t)n_shard * dtype_bytes(dtype));
    return probe_common(src, dtype, n_valid, flag, ctl, l2sq);
}

float orc_f16_to_f32(uint16_t h);
float orc_bf16_to_f32(uint16_t h);

int elx_widen(const void* src, int dtype, float* dst, int64_t n, void* stream) {
    (void)stream;
    if (!src || !dst) return ELX_ERR_NULL;
    if (dtype != ELX_F16 && dtype != ELX_BF16) return ELX_ERR_DTYPE;
    if (n < 0) return ELX_ERR_SIZE;
    const uint16_t* in = (const uint16_t*)src;
    for (int64_t i = 0; i < n; ++i) dst[i] = dtype == ELX_F16 ? orc_f16_to_f32(in[i]) : orc_bf16_to_f32(in[i]);
    return ELX_OK;
}

int elx_narrow_epilogue(const float* src, void* dst, int dtype, int64_t n_shard, int64_t n_valid, uint32_t* flag,
                        ElxCtl* ctl, void* stream) {
    (void)stream;
    if (!src || !dst) return ELX_ERR_NULL;
    if (dtype != ELX_F16 && dtype != ELX_BF16) return ELX_ERR_DTYPE;
    if (n_shard < 0 || n_valid < 0 || n_valid > n_shard) return ELX_ERR_SIZE;
    orc_cast(src, dst, dtype, n_shard);
    return probe_common(dst, dtype, n_valid, flag, ctl, 0);
}

int elx_grad_check_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                         uint32_t* chunk_flags, ElxCtl* ctl, float* chunk_l2sq, float* total_l2sq, float* scratch,
                         int64_t scratch_elems, void* stream) {
    (void)n_tiles;
    (void)scratch;
    (void)scratch_elems;
    (void)stream;
    if (!descs) return ELX_ERR_NULL;
    double total = 0.0;
    for (int c = first; c < first + count; ++c) {
        if (descs[c].dtype != dtype) {
            if (ctl) ctl->status |= ELX_STAT_BAD_DESC;
            continue;
        }
        float l2 = 0.0f;
        int rc = probe_common(grad_of(&descs[c]), dtype, descs[c].n_valid, chunk_flags ? &chunk_flags[c] : 0, ctl,
                              (chunk_l2sq || total_l2sq) ? &l2 : 0);
        if (rc != ELX_OK) return rc;
        if (chunk_l2sq) chunk_l2sq[c] = l2;
        total += l2;
    }
    if (total_l2sq) *total_l2sq = (float)total;
    return ELX_OK;
}

static void step_one(const ElxChunkDesc* d, const ElxSeg* segs, const ElxHyper* hyper, int n_groups,
                     const ElxCtl* ctl) {
    if (!ctl->skip) {
        for (int s = d->seg_first; s < d->seg_first + d->seg_count; ++s) {
            if (segs[s].group < 0 || segs[s].group >= n_groups) continue;
            orc_adam_f64(d->master, d->exp_avg, d->exp_avg_sq, grad_of(d), d->dtype, segs[s].begin, segs[s].end,
                         hyper[segs[s].group], ctl->step, ctl->div_scale);
        }
    }
    orc_cast(d->master, d->grad_param, d->dtype, d->n_shard);
}

int elx_adam_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype, const ElxSeg* segs,
                   const ElxHyper* hyper, int n_groups, ElxCtl* ctl, void* stream) {
    (void)n_tiles;
    (void)stream;
    if (!descs || !ctl) return ELX_ERR_NULL;
    if (n_groups > 64) return ELX_ERR_CAPACITY;
    for (int c = first; c < first + count; ++c) {
        if (descs[c].dtype != dtype) {
            ctl->status |= ELX_STAT_BAD_DESC;
            continue;
        }
        step_one(&descs[c], segs, hyper, n_groups, ctl);
    }
    return ELX_OK;
}

int elx_adam_chunk(float* master, float* exp_avg, float* exp_avg_sq, void* grad_param, int dtype, int64_t n_valid,
                   int64_t n_shard, ElxHyper hyper, ElxCtl* ctl, void* stream) {
    (void)stream;
    if (!master || !exp_avg || !exp_avg_sq || !grad_param || !ctl) return ELX_ERR_NULL;
    if (n_valid < 0 || n_valid > n_shard) return ELX_ERR_SIZE;
    ElxChunkDesc d;
    memset(&d, 0, sizeof(d));
    d.master = master;
    d.exp_avg = exp_avg;
    d.exp_avg_sq = exp_avg_sq;
    d.grad_param = grad_param;
    d.n_shard = n_shard;
    d.n_valid = n_valid;
    d.seg_count = n_valid > 0 ? 1 : 0;
    d.dtype = dtype;
    ElxSeg seg = {0, n_valid, 0, 0};
    step_one(&d, &seg, &hyper, 1, ctl);
    return ELX_OK;
}

int elx_cast_copyback(const float* master, void* dst, int dtype, int64_t n, void* stream) {
    (void)stream;
    if (!master || !dst) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    orc_cast(master, dst, dtype, n);
    return ELX_OK;
}

/* The NVLink entry points have no host-memory form: they need peer-mapped device memory. */
int elx_enable_peer_access(int peer_device) {
    (void)peer_device;
    return ELX_ERR_NODEVICE;
}
int elx_peer_barrier(ElxPeerTable flags, uint32_t epoch, ElxCtl* ctl, int exchange_overflow, int timeout_ms,
                     void* stream) {
    (void)flags; (void)epoch; (void)ctl; (void)exchange_overflow; (void)timeout_ms; (void)stream;
    return ELX_ERR_NODEVICE;
}
int elx_pull_reduce_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                          ElxPeerTable grads, const int64_t* block_off, const int64_t* stage_off,
                          uint32_t* chunk_flags, ElxCtl* ctl, void* stream) {
    (void)descs; (void)first; (void)count; (void)n_tiles; (void)dtype; (void)grads; (void)block_off; (void)stage_off;
    (void)chunk_flags; (void)ctl; (void)stream;
    return ELX_ERR_NODEVICE;
}
int elx_adam_multi_shadow(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                          int64_t n_tiles, int dtype, const ElxSeg* segs, const ElxHyper* hyper, int n_groups,
                          ElxCtl* ctl, void* stream) {
    (void)n_tiles;
    (void)stream;
    if (!descs || !shadow || !ctl) return ELX_ERR_NULL;
    if (n_groups > 64) return ELX_ERR_CAPACITY;
    for (int c = first; c < first + count; ++c) {
        const ElxChunkDesc* d = &descs[c];
        const ElxChunkDesc* o = &shadow[c];
        if (d->dtype != dtype || o->n_shard != d->n_shard) {
            ctl->status |= ELX_STAT_BAD_DESC;
            continue;
        }
        if (ctl->skip) {
            orc_cast(d->master, d->grad_param, d->dtype, d->n_shard);
            continue;
        }
        for (int s = d->seg_first; s < d->seg_first + d->seg_count; ++s) {
            if (segs[s].group < 0 || segs[s].group >= n_groups) continue;
            const int64_t b = segs[s].begin, n = segs[s].end - segs[s].begin;
            memcpy(o->master + b, d->master + b, (size_t)n * sizeof(float));
            memcpy(o->exp_avg + b, d->exp_avg + b, (size_t)n * sizeof(float));
            memcpy(o->exp_avg_sq + b, d->exp_avg_sq + b, (size_t)n * sizeof(float));
            orc_adam_f64(o->master, o->exp_avg, o->exp_avg_sq, grad_of(d), d->dtype, segs[s].begin, segs[s].end,
                         hyper[segs[s].group], ctl->step, ctl->div_scale);
        }
        orc_cast(o->master, d->grad_param, d->dtype, d->n_shard);
    }
    return ELX_OK;
}

/* ---- single-pass step over two sets of state (one rank; the collective form needs NVLink) ---- */

static void forced_skip(ElxCtl* ctl) {
    ctl->skip = 1;
    ctl->skipped_steps += 1;
    ctl->forced_skips += 1;
    ctl->div_scale = -1.0f;
    ctl->inv_div = 0.0f;
    ctl->found_inf = 0;
}

int elx_step_begin_optimistic(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags, void* stream) {
    (void)stream;
    if (!ctl) return ELX_ERR_NULL;
    if (cfg.max_norm > 0.0f) return ELX_ERR_ARG;
    ctl->repair = 0;
    if (ctl->status & ELX_STAT_TIMEOUT) {
        forced_skip(ctl);
        ctl->spec_state = 2;
    } else if (ctl->found_inf) {
        orc_step_begin(ctl, cfg, 0);
        ctl->spec_state = 2;
    } else {
        ctl->saved_scale = ctl->scale;
        ctl->saved_growth_step = ctl->growth_step;
        ctl->saved_hysteresis_step = ctl->hysteresis_step;
        ctl->saved_step = ctl->step;
        orc_step_begin(ctl, cfg, 0);
        ctl->spec_state = 1;
    }
    for (int i = 0; chunk_flags && i < n_chunk_flags; ++i) chunk_flags[i] = 0;
    return ELX_OK;
}

int elx_step_commit(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags, void* stream) {
    (void)stream;
    if (!ctl) return ELX_ERR_NULL;
    if (ctl->spec_state == 1) {
        const int expired = (ctl->status & ELX_STAT_TIMEOUT) != 0;
        if (expired || ctl->found_inf) {
            ctl->scale = ctl->saved_scale;
            ctl->growth_step = ctl->saved_growth_step;
            ctl->hysteresis_step = ctl->saved_hysteresis_step;
            ctl->step = ctl->saved_step;
            if (expired) {
                forced_skip(ctl);
            } else {
                ctl->found_inf = 1;
                orc_step_begin(ctl, cfg, 0);
            }
            ctl->repair = 1;
        } else {
            ctl->cur_set ^= 1u;
        }
    }
    ctl->spec_state = 0;
    ctl->found_inf = 0;
    for (int i = 0; chunk_flags && i < n_chunk_flags; ++i) chunk_flags[i] = 0;
    return ELX_OK;
}

int elx_adam_multi_single_pass(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                               int64_t n_tiles, int dtype, const ElxSeg* segs, const ElxHyper* hyper, int n_groups,
                               ElxCtl* ctl, uint32_t* chunk_flags, ElxPeerTable grads, ElxPeerTable gather,
                               const int64_t* block_off, const void* grads_mc, void* gather_mc, void* stream) {
    (void)n_tiles; (void)grads; (void)block_off; (void)stream;
    if (!descs || !shadow || !ctl) return ELX_ERR_NULL;
    if (gather.world > 0 || grads_mc || gather_mc) return ELX_ERR_NODEVICE;
    if (n_groups > 64) return ELX_ERR_CAPACITY;
    const ElxChunkDesc* src = ctl->cur_set ? shadow : descs;
    const ElxChunkDesc* dst = ctl->cur_set ? descs : shadow;
    for (int c = first; c < first + count; ++c) {
        const ElxChunkDesc* d = &src[c];
        const ElxChunkDesc* o = &dst[c];
        if (d->dtype != dtype || o->n_shard != d->n_shard) {
            ctl->status |= ELX_STAT_BAD_DESC;
            continue;
        }
        if (ctl->skip) {
            orc_cast(d->master, d->grad_param, d->dtype, d->n_shard);
            continue;
        }
        if (orc_probe(grad_of(d), d->dtype, d->n_valid)) {
            ctl->found_inf = 1;
            if (chunk_flags) chunk_flags[c] = 1;
        }
        for (int s = d->seg_first; s < d->seg_first + d->seg_count; ++s) {
            if (segs[s].group < 0 || segs[s].group >= n_groups) continue;
            const int64_t b = segs[s].begin, n = segs[s].end - segs[s].begin;
            memcpy(o->master + b, d->master + b, (size_t)n * sizeof(float));
            memcpy(o->exp_avg + b, d->exp_avg + b, (size_t)n * sizeof(float));
            memcpy(o->exp_avg_sq + b, d->exp_avg_sq + b, (size_t)n * sizeof(float));
            orc_adam_f64(o->master, o->exp_avg, o->exp_avg_sq, grad_of(d), d->dtype, segs[s].begin, segs[s].end,
                         hyper[segs[s].group], ctl->step, ctl->div_scale);
        }
        orc_cast(o->master, d->grad_param, d->dtype, d->n_shard);
    }
    return ELX_OK;
}

int elx_adam_multi_repair(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count, int64_t n_tiles,
                          int dtype, ElxCtl* ctl, ElxPeerTable gather, const int64_t* block_off, void* gather_mc,
                          void* stream) {
    (void)n_tiles; (void)dtype; (void)block_off; (void)gather_mc; (void)stream;
    if (!descs || !shadow || !ctl) return ELX_ERR_NULL;
    if (gather.world > 0) return ELX_ERR_NODEVICE;
    if (!ctl->repair) return ELX_OK;
    const ElxChunkDesc* src = ctl->cur_set ? shadow : descs;
    for (int c = first; c < first + count; ++c) orc_cast(src[c].master, src[c].grad_param, src[c].dtype, src[c].n_shard);
    return ELX_OK;
}

int elx_adam_multi_hostmem(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                           const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl, void* stream) {
    return elx_adam_multi(descs, first, count, n_tiles, dtype, segs, hyper, n_groups, ctl, stream);
}

int elx_adam_multi_push(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                        const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl, ElxPeerTable gather,
                        const int64_t* block_off, void* stream) {
    (void)descs; (void)first; (void)count; (void)n_tiles; (void)dtype; (void)segs; (void)hyper; (void)n_groups;
    (void)ctl; (void)gather; (void)block_off; (void)stream;
    return ELX_ERR_NODEVICE;
}
int elx_adam_multi_pull_push(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                             const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl, ElxPeerTable grads,
                             ElxPeerTable gather, const int64_t* block_off, void* stream) {
    (void)descs; (void)first; (void)count; (void)n_tiles; (void)dtype; (void)segs; (void)hyper; (void)n_groups;
    (void)ctl; (void)grads; (void)gather; (void)block_off; (void)stream;
    return ELX_ERR_NODEVICE;
}
int elx_multimem_reduce(const void* src_mc, void* dst, int dtype, int64_t n, void* stream) {
    (void)src_mc; (void)dst; (void)dtype; (void)n; (void)stream;
    return ELX_ERR_NODEVICE;
}
int elx_ipc_open(const void* handle, void** base) {
    (void)handle; (void)base;
    return ELX_ERR_NODEVICE;
}
int elx_ipc_close(void* base) {
    (void)base;
    return ELX_ERR_NODEVICE;
}
int elx_peek_u32(const void* device_ptr, uint32_t* value) {
    if (!device_ptr || !value) return ELX_ERR_NULL;
    *value = *(const uint32_t*)device_ptr;
    return ELX_OK;
}
int elx_peer_alloc(int64_t bytes, void** ptr, void* handle) {
    (void)bytes; (void)ptr; (void)handle;
    return ELX_ERR_NODEVICE;
}
int elx_peer_free(void* ptr) {
    (void)ptr;
    return ELX_ERR_NODEVICE;
}
int elx_copy_async(void* dst, const void* src, int64_t bytes, void* stream) {
    (void)stream;
    if (!dst || !src) return ELX_ERR_NULL;
    memmove(dst, src, (size_t)bytes);
    return ELX_OK;
}
