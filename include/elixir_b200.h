/*
 * elixir_b200 — C ABI of the chunk-level mixed-precision optimizer step for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host runtime binds to (ctypes / cffi / pybind / plain C).  Every pointer
 * marked "device" is a CUDA device pointer owned by the caller; on the step path the library never
 * allocates, frees or synchronises (the set-up calls of the NVLink section are the exception:
 * elx_peer_alloc / elx_peer_free allocate and free, elx_peek_u32 blocks).  Every entry point is
 * stream-ordered on the `stream` it is given (a cudaStream_t passed as void*, NULL = the legacy default
 * stream) and returns an `int` status: 0 on success, a negative ELX_ERR_* code when an argument is
 * rejected (nothing was launched) or a launch failed.
 *
 * The functions replace the following pieces of hpcaitech/Elixir (paths inside that project):
 *   elixir/wrapper/optimizer.py   ElixirOptimizer.step / _check_overflow / _get_combined_scale
 *   elixir/chunk/core/chunk.py    Chunk.reduce (copy into the shard), set_overflow_flag,
 *                                 set_l2_norm, optim_update
 *   colossalai FusedAdam/HybridAdam.step(div_scale=...) and DynamicGradScaler.update(...)
 *   (third-party to Elixir, called at elixir/wrapper/optimizer.py:78-86,198,208,216)
 */
#ifndef ELIXIR_B200_H
#define ELIXIR_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ELX_ABI_VERSION 2

/* Elements per work tile.  `ElxChunkDesc.tile_begin` counts tiles of this many elements. */
#define ELX_TILE 4096

/* dtype codes for the low-precision (working / gradient) chunk. */
#define ELX_F16 0
#define ELX_BF16 1
#define ELX_F32 2

/* status codes */
#define ELX_OK 0
#define ELX_ERR_NULL (-1)      /* a required pointer is NULL                                   */
#define ELX_ERR_ALIGN (-2)     /* a pointer is not aligned as documented                        */
#define ELX_ERR_SIZE (-3)      /* negative size, n_valid > n_shard, count out of range ...      */
#define ELX_ERR_DTYPE (-4)     /* unknown dtype code                                            */
#define ELX_ERR_LAUNCH (-5)    /* the CUDA runtime rejected the launch (see elx_last_cuda_error) */
#define ELX_ERR_ARG (-6)       /* inconsistent argument combination                             */
#define ELX_ERR_NODEVICE (-7)  /* no usable CUDA device / driver                                */
#define ELX_ERR_CAPACITY (-8)  /* request exceeds a documented fixed capacity                   */

/* sticky bits in ElxCtl.status */
#define ELX_STAT_LATE_INF 1u   /* the Adam kernel met a non-finite gradient the probe had not flagged */
#define ELX_STAT_BAD_DESC 2u   /* a kernel could not map a tile to a chunk descriptor                   */
#define ELX_STAT_TIMEOUT 4u    /* a bounded wait (on-chip barrier or another rank) expired; the kernel gave up.
                                  While the bit is set elx_step_begin decides "skip" and leaves the loss
                                  scaler alone: parameters are never updated from data that may be incomplete */

/*
 * Device-resident control block of one optimizer (128 bytes, 16-byte aligned).  It replaces the
 * host-side state that the reference reads back with .item() on every step: the loss scale and
 * its counters (DynamicGradScaler), the per-chunk overflow booleans OR-ed by
 * ElixirOptimizer._check_overflow (optimizer.py:137-142), and the per-tensor Adam step count.
 */
typedef struct ElxCtl {
    float    scale;            /* current loss scale                                             */
    uint32_t found_inf;        /* OR of all probes since the last elx_step_begin                  */
    int32_t  growth_step;      /* clean steps since the last growth / overflow                    */
    int32_t  hysteresis_step;  /* overflows seen since the last growth                            */
    int32_t  step;             /* number of applied (non-skipped) Adam steps                      */
    uint32_t skip;             /* decision of the last elx_step_begin: 1 = copy-back only         */
    float    div_scale;        /* divisor for the gradients of this step, -1 = do not divide      */
    float    inv_div;          /* 1/div_scale when that product is exact (power of two), else 0   */
    uint32_t skipped_steps;    /* total skipped steps                                             */
    uint32_t status;           /* sticky ELX_STAT_* bits                                          */
    uint32_t late_inf;         /* set by the Adam kernel when it meets inf/nan on an applied step */
    uint32_t forced_skips;     /* steps skipped because ELX_STAT_TIMEOUT was set, not for an overflow */
    float    clip_coef;        /* clip factor of the last applied step (1 = not clipped)          */
    float    grad_norm;        /* unscaled global gradient norm of the last applied step          */
    /* single-pass (two-set) step, see elx_step_begin_optimistic: */
    uint32_t cur_set;          /* which of the two sets of master/moment arrays is the current one */
    uint32_t spec_state;       /* 0 idle, 1 optimistic decision pending its commit, 2 decided up front */
    uint32_t repair;           /* set by elx_step_commit when the working copies must be rebuilt   */
    float    saved_scale;      /* scaler state as it was before the optimistic decision            */
    int32_t  saved_growth_step;
    int32_t  saved_hysteresis_step;
    int32_t  saved_step;
    uint32_t reserved[11];
} ElxCtl;

/* Loss-scaler configuration, passed by value.  Mirrors DynamicGradScaler / ConstantGradScaler as
 * constructed at elixir/wrapper/optimizer.py:76-86. */
typedef struct ElxScalerCfg {
    int32_t dynamic;           /* 1 = dynamic scaler, 0 = constant scale (never updated)          */
    float   growth_factor;
    float   backoff_factor;
    float   min_scale;         /* <= 0: no lower bound                                            */
    float   max_scale;         /* <= 0: no upper bound                                            */
    int32_t growth_interval;
    int32_t hysteresis;
    float   max_norm;          /* > 0 enables gradient clipping by global L2 norm                 */
} ElxScalerCfg;

/* Hyper-parameters of one optimizer param group (host-written device table, 32 bytes each). */
typedef struct ElxHyper {
    float   lr;
    float   beta1;
    float   beta2;
    float   eps;
    float   weight_decay;
    int32_t adamw_mode;        /* 1 = decoupled decay (AdamW), 0 = L2 (decay added to the gradient) */
    int32_t bias_correction;   /* 0 = both corrections are 1                                        */
    int32_t reserved;
} ElxHyper;

/* A contiguous range [begin, end) of a shard whose elements belong to param group `group`.
 * Segments of one chunk are sorted, disjoint and lie inside [0, n_valid).  Elements of the shard
 * covered by no segment are not updated (their working copy is still refreshed from the master).
 * Equivalent of ElixirOptimizer.param_to_range (optimizer.py:238-265) with neighbours merged. */
typedef struct ElxSeg {
    int64_t begin;
    int64_t end;
    int32_t group;
    int32_t reserved;
} ElxSeg;

/* One chunk shard of this rank (device table, 80 bytes each): the fp32 master chunk's shard, the
 * two Adam moments laid out congruently, and the paired low-precision shard that holds the
 * gradient before the step and the refreshed working copy after it (optimizer.py:115-124,
 * chunk.py:403-415).  All pointers must be 32-byte aligned.
 * grad_src separates the two roles of the low-precision shard: when it is not NULL the probe and the
 * update READ the gradient there (n_shard elements of `dtype`, e.g. the block autograd filled) and
 * only WRITE the refreshed working copy to grad_param, so that no copy into the shard is needed
 * before the step (the copy that ends Chunk.reduce at world size 1, chunk.py:310-313).  After the
 * step the shard holds parameters either way. */
typedef struct ElxChunkDesc {
    float*  master;            /* device, n_shard floats                                           */
    float*  exp_avg;           /* device, n_shard floats                                           */
    float*  exp_avg_sq;        /* device, n_shard floats                                           */
    void*   grad_param;        /* device, n_shard elements of `dtype`: gradient in, working copy out */
    int64_t n_shard;           /* shard_size                                                       */
    int64_t n_valid;           /* valid_end: elements that hold real parameters (chunk.py:253-257) */
    int64_t tile_begin;        /* sum over earlier descriptors of ceil(n_shard / ELX_TILE)         */
    int32_t seg_first;         /* index of this chunk's first segment in the segment table         */
    int32_t seg_count;
    int32_t dtype;             /* ELX_F16 / ELX_BF16 / ELX_F32                                      */
    int32_t reserved;
    const void* grad_src;      /* device, n_shard elements of `dtype`, or NULL = the gradient is in grad_param */
} ElxChunkDesc;

/* Device addresses of one buffer per rank of a single-node group, as seen from THIS process: entry j
 * is rank j's buffer mapped into this process (peer-mapped / IPC memory; entry `rank` is the local
 * one).  All are 32-byte aligned. */
#define ELX_MAX_PEERS 16
typedef struct ElxPeerTable {
    void*   base[ELX_MAX_PEERS];
    int32_t rank;
    int32_t world;
} ElxPeerTable;

/* ---- library ----------------------------------------------------------------------------- */

/* ABI version of the loaded library (ELX_ABI_VERSION it was built with). */
int elx_version(void);

/* Static, human-readable text for a status code. */
const char* elx_strerror(int status);

/* Text of the last CUDA runtime error seen by this thread inside the library ("" if none). */
const char* elx_last_cuda_error(void);

/* Launch-shape knobs, by name; a negative value restores the default.  Affects later launches of
 * the calling process; results never depend on them (bit-identical for every setting except
 * math_mode).
 *   "adam_threads"       direct variant: 256 (16 elements per thread) or 512 (8 per thread)
 *   "adam_ctas_per_sm"   direct variant: cap on the persistent grid, 0 = every resident CTA
 *   "probe_ctas_per_sm"  the same for the probe kernels
 *   "probe_unroll"       4 or 8 tiles in flight per probe CTA
 *   "probe_variant"      elx_grad_check without a norm: 0 = per-thread loads, 1 = a bulk-copy ring through
 *                        shared memory for arrays of 16 MiB and more that start on a 16-byte boundary
 *                        (default), 2 = the ring for every such array whatever its size
 *   "adam_variant"       0 = direct 256-bit global accesses, 1 = bulk-copy (TMA) pipeline through
 *                        shared memory
 *   "pull_ctas_per_sm"   cap on the grid of the pull reduce-scatter kernel, 0 = every resident CTA
 *   "pull_variant"       0 = per-lane peer loads, 1 = bulk-copy staging through shared memory (16-bit
 *                        chunks and groups of 2, 4 or 8 ranks; other cases use variant 0)
 *   "adam_tma_ctas"      grid of the bulk-copy update kernel, 0 = one CTA per SM; with "pull_tma_ctas" (the
 *                        same for the bulk-copy pull kernel, which then also uses a deeper shared-memory ring,
 *                        since few CTAs have to keep more data in flight each) it splits the SMs between an
 *                        update and a pull that run at the same time on two streams
 *   "adam_tma_stages"    ring depth of the bulk-copy update kernel: 0 = the deepest that fits in shared memory
 *                        (four 56 KB stages for 16-bit chunks in IEEE mode, else three), 3 = three
 *   "math_mode"          1 = IEEE division and square root in the update, 2 = reciprocal
 *                        multiplies and approximate division (both within 1e-6 relative) */
int elx_set_tuning(const char* name, int value);

/* Number of floats of scratch the probe entry points need for `n_tiles` tiles when an L2 norm is
 * requested (one partial sum per tile). */
int64_t elx_probe_scratch_elems(int64_t n_tiles);

/* ---- control block ------------------------------------------------------------------------ */

/* Initialise a device control block: scale = initial_scale, all counters and flags zero.
 * Replaces DynamicGradScaler.__init__ state.  ctl: device, 16-byte aligned. */
int elx_ctl_init(ElxCtl* ctl, float initial_scale, void* stream);

/*
 * The per-step decision, entirely on the device (one tiny launch, no host read-back).  Replaces the
 * head of ElixirOptimizer.step (optimizer.py:192-209):
 *   found_inf = OR of chunk overflow flags            (_check_overflow, :137-142)
 *   if found_inf: skip = 1, scaler.update(True)        (:196-203)
 *   else: div = loss scale read BEFORE the update, times the clip factor when clipping is on and
 *         the factor exceeds 1, or -1 when div == 1    (_get_combined_scale, :166-183)
 *         scaler.update(False); step += 1              (:208, optimizer state['step'])
 *   found_inf and the per-chunk overflow words are cleared   (_clear_optim_states, :144-147)
 * norm_sq: device pointer to the global sum of squared (still scaled) gradients, or NULL when
 * cfg.max_norm <= 0.  chunk_flags: device array of n_chunk_flags per-chunk overflow words
 * (Chunk.overflow) to clear, or NULL.
 * While ELX_STAT_TIMEOUT is set in ctl->status the decision is "skip" whatever found_inf says, the
 * loss scaler and the step count are left alone and ctl->forced_skips is incremented.
 */
int elx_step_begin(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq, uint32_t* chunk_flags,
                   int n_chunk_flags, void* stream);

/* ---- overflow / norm probe ------------------------------------------------------------------ */

/*
 * Probe one gradient shard: set *flag (and ctl->found_inf when ctl != NULL) to 1 if any of the
 * first n_valid elements is inf or nan, tested on the exponent bits of the stored low-precision
 * values.  Replaces Chunk.set_overflow_flag (chunk.py:214-216) as used by
 * update_extra_reduce_info (chunk.py:345-356).  The flag is only ever raised, never cleared.
 * When l2sq != NULL the sum of squares of the same elements (each converted to fp32) is written
 * to *l2sq, reduced in a fixed order (bit-reproducible); replaces set_l2_norm (chunk.py:218-221).
 * That needs `scratch` (device floats, >= elx_probe_scratch_elems(ceil(n_valid/ELX_TILE))).
 * g: device, aligned to its element size (32-byte alignment enables the vector path).  flag, l2sq may
 * alias nothing else.
 */
int elx_grad_check(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl,
                   float* l2sq, float* scratch, int64_t scratch_elems, void* stream);

/*
 * elx_grad_check without a scratch argument, for callers that have no way to hand the library device
 * memory of their own: a host runtime that binds only this C ABI and owns no allocator, or code that
 * runs where cudaMalloc is off limits (inside a library callback, on a thread that must not block
 * on the allocator's lock, in a process whose memory pool is already carved up).  It has no
 * counterpart in the reference, whose norm goes through torch temporaries.
 *
 * The per-tile partial sums go to a 64 KiB array that is part of the library image on every GPU that
 * loads it, so with l2sq != NULL n_valid is limited to elx_grad_check_static_max_elems() (67 108 864)
 * elements; a larger request returns ELX_ERR_CAPACITY and launches nothing (without l2sq no scratch is
 * used and any size is accepted).  The call allocates and frees nothing.
 * The first call on each device (with l2sq != NULL) looks up the array's device address once and
 * caches it for the life of the process (the cache does not survive cudaDeviceReset); make that first
 * call outside any stream capture, with the device current.
 * All calls on a device share the array and every call overwrites the slots it uses (nothing has to
 * start at zero), so two calls whose kernels can overlap on the GPU (different streams without an
 * ordering between them) race on it: keep calls on one device ordered.
 * Results are bit-identical to elx_grad_check given the same inputs.
 */
int elx_grad_check_static(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl,
                          float* l2sq, void* stream);

/* Largest n_valid elx_grad_check_static accepts. */
int64_t elx_grad_check_static_max_elems(void);

/*
 * The same probe fused with the copy that ends Chunk.reduce (chunk.py:313, 484-489): copies
 * n_shard elements src -> dst (the reduced slice of the replicated block into the persistent
 * shard) and probes the first n_valid of them in the same pass.  src, dst: device, aligned to the
 * element size (32-byte alignment of both enables the vector path), must not overlap.
 */
int elx_reduce_epilogue(const void* src, void* dst, int dtype, int64_t n_shard, int64_t n_valid,
                        uint32_t* flag, ElxCtl* ctl, float* l2sq, float* scratch,
                        int64_t scratch_elems, void* stream);

/*
 * The two ends of a gradient reduction carried out in fp32 (Chunk.reduce with always_fp32,
 * chunk.py:288-308: widen the low-precision block, divide and reduce-scatter in fp32, write the average
 * back in the chunk dtype).
 * elx_widen: dst[i] = float(src[i]) for i in [0, n); dtype is ELX_F16 or ELX_BF16.
 * elx_narrow_epilogue: dst[i] = src[i] rounded to nearest-even in `dtype` for i in [0, n_shard) -- the
 * fp32 average of this rank's slice into its persistent shard -- and the rounded values of [0, n_valid)
 * are probed as elx_grad_check does (the copy ending Chunk.reduce and update_extra_reduce_info in one pass).
 * Pointers need element alignment; 32-byte alignment of both enables the vector path.
 */
int elx_widen(const void* src, int dtype, float* dst, int64_t n, void* stream);
int elx_narrow_epilogue(const float* src, void* dst, int dtype, int64_t n_shard, int64_t n_valid,
                        uint32_t* flag, ElxCtl* ctl, void* stream);

/*
 * Probe descriptors [first, first + count) of a descriptor table in ONE launch.  chunk_flags
 * (device, one uint32 per descriptor of the table, may be NULL) receives the per-chunk overflow
 * booleans (Chunk.overflow); ctl->found_inf receives their OR.  When chunk_l2sq != NULL it
 * receives one sum of squares per descriptor (Chunk.l2_norm) and total_l2sq (may be NULL) their
 * sum in descriptor order.  n_tiles = number of ELX_TILE tiles of the probed descriptors; dtype =
 * the dtype every probed descriptor carries (a descriptor with another dtype is left untouched and
 * raises ELX_STAT_BAD_DESC in ctl->status).
 */
int elx_grad_check_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles,
                         int dtype, uint32_t* chunk_flags, ElxCtl* ctl, float* chunk_l2sq, float* total_l2sq,
                         float* scratch, int64_t scratch_elems, void* stream);

/* ---- fused update ---------------------------------------------------------------------------- */

/*
 * The fused step over descriptors [first, first + count): for every element of every segment
 *   g = float(g_lowp);  g = g / ctl->div_scale (when > 0);  Adam / AdamW on master, exp_avg,
 *   exp_avg_sq with the group's hyper-parameters and bias corrections for ctl->step;
 * then, over the WHOLE shard [0, n_shard), the working copy is refreshed with the master rounded
 * to nearest-even.  When ctl->skip is 1 only the refresh runs.  One pass over memory: 28 bytes per
 * element with 16-bit gradients.  Replaces _set_grad_ptr + optim.step(div_scale) +
 * _update_fp16_params (optimizer.py:115-135, 216-219; chunk.py:403-415).
 * n_tiles = number of ELX_TILE tiles of those descriptors; dtype = the dtype all of them carry.
 * hyper: device table of n_groups entries (n_groups <= 64).  All tables are device memory.
 */
int elx_adam_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                   const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl,
                   void* stream);

/*
 * elx_adam_multi for shards kept in page-locked host memory that is mapped into the device's address
 * space (cudaHostAlloc / torch pinned memory: under unified addressing the host pointer is the device
 * pointer) -- the reference's `shard_device=cpu` placement (chunk.py:101-111), where HybridAdam runs its
 * CPU kernel on such shards (optimizer.py:19, 216).  Here the same GPU kernel updates them in place over
 * PCIe: no host arithmetic, no staging copies, 14 bytes per element in each direction with 16-bit
 * gradients.  Same arguments, results and status codes as elx_adam_multi; the master / exp_avg /
 * exp_avg_sq / grad_param pointers of the descriptors may be any mix of device and mapped host memory,
 * the tables (descs, segs, hyper, ctl) are device memory.  Always runs the direct load/store variant of
 * the update (the bulk-copy pipeline is kept to device memory).
 */
int elx_adam_multi_hostmem(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                           const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl,
                           void* stream);

/*
 * elx_adam_multi out of place: the updated master and moments of descriptor c are written to the arrays of
 * shadow[c] (same n_shard and tile_begin; its grad_param is ignored) while descs[c]'s arrays are only read;
 * the refreshed working copy still replaces the gradients in descs[c].grad_param.  Elements no segment
 * covers are not written, so both sets must start out equal.  No counterpart in the reference: it lets a
 * host start updating before the last gradient has arrived (elx_step_begin called on the assumption of no
 * overflow) and drop the result, by not swapping the two sets, when an overflow turns up afterwards --
 * the reference's rule that one overflow skips every parameter (optimizer.py:194-203) then still holds.
 * Always runs the bulk-copy variant.  A skipped step (ctl->skip) refreshes the working copy from descs as
 * elx_adam_multi does and writes nothing to the shadow set.
 * The arrays of both tables must be device memory: this entry point, elx_adam_multi_push and the single-pass
 * entry points always move tiles with bulk copies, which are kept to device memory (shards in mapped host
 * memory go through elx_adam_multi_hostmem); the library cannot tell where an array lives from a table in device
 * memory, so the caller has to keep to this.
 */
int elx_adam_multi_shadow(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                          int64_t n_tiles, int dtype, const ElxSeg* segs, const ElxHyper* hyper,
                          int n_groups, ElxCtl* ctl, void* stream);

/* ---- single-pass step over two sets of state ---------------------------------------------------- */

/*
 * The step as ONE pass over memory: unscale, inf/nan detection, Adam / AdamW and the rounded working copy in
 * the same kernel, 28 bytes per element with 16-bit gradients and no separate probe.  The reference's rule
 * that one overflow anywhere skips every parameter (optimizer.py:194-203) is kept by updating OUT OF PLACE:
 * the state exists twice (descs = set 0, shadow = set 1, congruent tables as for elx_adam_multi_shadow; 12
 * bytes per element more memory), the kernel reads the current set (ElxCtl.cur_set) and writes the other one,
 * and the sets change roles only when the whole step turned out clean.  Nothing is read back by the host:
 *
 *   elx_step_begin_optimistic   decision on the assumption of no overflow: divisor from the current loss scale,
 *                               scaler "clean step" update, step count (the state before it is kept in the
 *                               control block).  An overflow already pending in found_inf, or a set
 *                               ELX_STAT_TIMEOUT, is decided here for real (skip), as elx_step_begin would.
 *                               Gradient clipping needs the global norm first and is not available here.
 *   elx_adam_multi_single_pass  per element of every segment the update of elx_adam_multi, written to the other
 *                               set; every gradient element of [0, n_valid) it reads is tested for inf/nan
 *                               (chunk_flags, ctl->found_inf).  May be launched chunk by chunk.  When the step
 *                               was decided as skipped up front it only refreshes the working copies.
 *   [W > 1: elx_peer_barrier with exchange_overflow, so that every rank commits the same way]
 *   elx_step_commit             clean: cur_set flips.  Overflow: the saved scaler state comes back, the overflow
 *                               branch of elx_step_begin runs on it (skip, back-off), cur_set stays, and
 *                               ctl->repair is set.  found_inf and chunk_flags are cleared.
 *   elx_adam_multi_repair       returns at once unless ctl->repair is set; then rebuilds the working copies
 *                               (and re-sends them to the gather blocks) from the current, untouched set.
 *
 * With grads_mc / gather_mc (multicast addresses of the ranks' gradient and gather slabs in one NVLink domain,
 * from a multicast object bound to all of them) the kernel also carries both collectives of the sharded step:
 * the gradient tile of this rank's shard is fetched as the sum over all ranks, added up inside the switch
 * (multimem.ld_reduce, fp32 accumulation, one rounding to the chunk dtype) and multiplied by 1/W, and the
 * refreshed working-copy tile is stored once to the multicast address (multimem.st), which delivers it to every
 * rank's gather block -- reduce-scatter (Chunk.reduce, chunk.py:282-315), update and all-gather
 * (Chunk.__update_replica, chunk.py:475-482) tile by tile in one launch, with about (W + 1) / W of a chunk's
 * bytes on each direction of the links instead of 2 (W - 1) / W.  The reduced gradient is never written to
 * memory.  The overflow test then sees the rounded SUM: a sum that leaves the range of fp16 while the average
 * would not is treated as an overflow (a skipped step and a scale back-off), where the reference, which divides
 * before it sums, would have applied the step.  grads / gather are the same slabs as peer tables (for ragged
 * tiles, which use plain peer accesses); block_off as for elx_adam_multi_push.  All NULL / world 0: one rank,
 * gradients read from grad_src / grad_param.  gather given without the multicast addresses: the gradients are
 * read from the shard (where elx_pull_reduce_multi left the rank average) and the working copy is pushed to the
 * gather blocks with plain bulk stores, as elx_adam_multi_push does -- the out-of-place form of that entry
 * point, which lets the update of one chunk run while later chunks are still being reduced.
 */
int elx_step_begin_optimistic(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags,
                              void* stream);
int elx_step_commit(ElxCtl* ctl, ElxScalerCfg cfg, uint32_t* chunk_flags, int n_chunk_flags, void* stream);
int elx_adam_multi_single_pass(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                               int64_t n_tiles, int dtype, const ElxSeg* segs, const ElxHyper* hyper,
                               int n_groups, ElxCtl* ctl, uint32_t* chunk_flags, ElxPeerTable grads,
                               ElxPeerTable gather, const int64_t* block_off, const void* grads_mc,
                               void* gather_mc, void* stream);
int elx_adam_multi_repair(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                          int64_t n_tiles, int dtype, ElxCtl* ctl, ElxPeerTable gather,
                          const int64_t* block_off, void* gather_mc, void* stream);

/* ---- NVLink paths (single node, peer-mapped memory) -------------------------------------------- */

/* Enable access from the current device to memory of `peer_device` (cudaDeviceEnablePeerAccess;
 * "already enabled" is success). */
int elx_enable_peer_access(int peer_device);

/* The one place where the library allocates: a buffer of `bytes` on the current device that other
 * processes of the box can map (cudaMalloc + cudaIpcGetMemHandle).  `handle` receives the 64-byte
 * cudaIpcMemHandle_t to send to the peers.  Set-up time only; elx_peer_free releases the buffer. */
int elx_peer_alloc(int64_t bytes, void** ptr, void* handle);
int elx_peer_free(void* ptr);

/* Map a buffer another process exported (a 64-byte cudaIpcMemHandle_t) for access from the CURRENT device
 * of the calling process; *base receives the address of the exporter's allocation.  Open each handle
 * once per process.  elx_ipc_close unmaps it. */
int elx_ipc_open(const void* handle, void** base);
int elx_ipc_close(void* base);

/* Set-up check of a mapping: confirm that device_ptr is device memory known to this process and read one
 * word from it with a blocking copy.  Synchronises; not for the step path. */
int elx_peek_u32(const void* device_ptr, uint32_t* value);

/*
 * Barrier across the ranks of a box, on the device: rank r writes `epoch` into its slot of every
 * rank's flag region (flags.base[j], 256 zero-initialised uint32 each) and waits until every rank
 * has written `epoch` into r's region.  Everything a rank wrote to its peer-visible buffers before
 * the barrier is visible to every rank after it.  With exchange_overflow != 0 each rank's
 * ctl->found_inf rides along and ctl->found_inf becomes the OR over all ranks — the agreement the
 * reference lacks (elixir/wrapper/optimizer.py:137-142 decides per rank).  Epochs must increase by 1
 * per call, starting at 1, identically on all ranks.  The wait is bounded: after timeout_ms the kernel
 * raises ELX_STAT_TIMEOUT in ctl->status and returns.
 */
int elx_peer_barrier(ElxPeerTable flags, uint32_t epoch, ElxCtl* ctl, int exchange_overflow, int timeout_ms,
                     void* stream);

/*
 * Reduce-scatter by pulling, fused with the probe: for every descriptor c in [first, first + count)
 * this rank's shard (descs[c].grad_param, n_shard elements) becomes the rank average of slice
 * [rank * n_shard, (rank + 1) * n_shard) of chunk c's gradient block, read from every rank's slab
 * (grads.base[j] + block_off[c] elements): sum over j in rank order of float(x_j) * (1/W) in fp32, rounded
 * once to the chunk dtype; the first n_valid results are probed for inf/nan (chunk_flags[c],
 * ctl->found_inf).  Replaces Chunk.reduce + update_extra_reduce_info (elixir/chunk/core/chunk.py:282-315,
 * 345-356) for a group inside one NVLink domain; the reference's `x / W` then SUM differs from it
 * only in where the roundings fall.  Call it between two elx_peer_barrier calls: one after every rank
 * wrote its blocks, one before any rank overwrites them.
 * stage_off == NULL: every grads.base[j] is rank j's whole slab.  stage_off != NULL: grads.base[j] for
 * j != rank is a LOCAL buffer that already holds a copy of rank j's slice for this rank, chunk c's slice
 * starting at element stage_off[c]; grads.base[rank] is still this rank's own slab.
 */
int elx_pull_reduce_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                          ElxPeerTable grads, const int64_t* block_off, const int64_t* stage_off,
                          uint32_t* chunk_flags, ElxCtl* ctl, void* stream);

/*
 * dst[i] = the sum over all ranks of element i of the buffers behind the multicast address src_mc, formed by the
 * NVLink switch (multimem.ld_reduce with fp32 accumulation, returned in `dtype`, ELX_F16 or ELX_BF16): the
 * reduce-scatter of Chunk.reduce (chunk.py:299-303) without the division, for a caller that wants the reduced slice in
 * memory -- the single-pass kernel consumes the same values without storing them, and the parity tests use this entry
 * point to see them.  For more than two ranks the switch's result is not the rank-order fp32 sum rounded once: it can
 * differ from it in the last bit of the 16-bit format.  n a multiple of 8; src_mc and dst 16-byte aligned.
 */
int elx_multimem_reduce(const void* src_mc, void* dst, int dtype, int64_t n, void* stream);

/* One asynchronous device-to-device copy on `stream` (cudaMemcpyAsync, any mix of local and peer-mapped
 * addresses): the copy engines move whole slices over NVLink at a higher rate than SM-issued accesses.
 * Used by the staged form of the sharded step: the other ranks' slices are first copied into local
 * staging buffers, then elx_pull_reduce_multi runs with stage_off != NULL on local memory only. */
int elx_copy_async(void* dst, const void* src, int64_t bytes, void* stream);

/*
 * elx_adam_multi fused with the parameter all-gather: every refreshed low-precision tile is also
 * stored into every rank's gather slab at gather.base[j] + block_off[c] + rank * n_shard (elements),
 * so that after the next elx_peer_barrier each rank holds the whole updated chunk
 * (Chunk.__update_replica, chunk.py:475-482) without a separate all-gather pass.
 */
int elx_adam_multi_push(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                        const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl,
                        ElxPeerTable gather, const int64_t* block_off, void* stream);

/*
 * elx_adam_multi_push with the reduce-scatter inside as well: the gradient of a tile is not read from the shard
 * but fetched from every rank's gradient slab (grads.base[j] + block_off[c] + rank * n_shard, the slice
 * elx_pull_reduce_multi would read) with plain bulk loads into shared memory and averaged there exactly as
 * elx_pull_reduce_multi averages (fp32, rank order, one rounding to the chunk dtype), so that the links are busy
 * while the previous tile is being updated and the reduced gradient never touches memory: Chunk.reduce, the update
 * and __update_replica (chunk.py:282-315, 475-482; optimizer.py:115-135, 216) in one launch, in place.
 * An update in place needs the decision first: call it after elx_step_begin, with ctl->found_inf formed from the
 * INPUTS (elx_grad_check over this rank's own gradient slab, then elx_peer_barrier with exchange_overflow) --
 * the fp32-accumulated average is non-finite exactly when one of its inputs is.
 * 16-bit chunks; groups of two ranks (ELX_ERR_CAPACITY otherwise: the peers' slices of three tiles in flight have
 * to fit in shared memory beside the update's own stages).
 */
int elx_adam_multi_pull_push(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                             const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl,
                             ElxPeerTable grads, ElxPeerTable gather, const int64_t* block_off, void* stream);

/*
 * Single-shard convenience form with the hyper-parameters by value and one implicit segment
 * [0, n_valid).  Same arithmetic as elx_adam_multi.  Pointers need only be aligned to their
 * element size; the vector path is used when all of them are 32-byte aligned.
 */
int elx_adam_chunk(float* master, float* exp_avg, float* exp_avg_sq, void* grad_param, int dtype,
                   int64_t n_valid, int64_t n_shard, ElxHyper hyper, ElxCtl* ctl, void* stream);

/* Working-copy refresh alone: dst[i] = round_to_nearest_even(master[i]) for i in [0, n).
 * Replaces Chunk.optim_update for CUDA shards (chunk.py:413-415). */
int elx_cast_copyback(const float* master, void* dst, int dtype, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ELIXIR_B200_H */
