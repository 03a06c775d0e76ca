// Part of the elixir_b200 CUDA library (C ABI: include/elixir_b200.h).  See elx_common.cuh for the
// overview of the kernels and of how the sources are divided.
#include <type_traits>

#include "elx_common.cuh"

using namespace elx;

namespace {

// ------------------------------------------------------------------------------------------------
// Adam
// ------------------------------------------------------------------------------------------------

// Per-group constants derived once per CTA from ElxHyper and the device step counter.
struct GroupK {
    float lr, beta1, omb1, beta2, omb2, eps;
    float wd_l2;   // weight decay added to the gradient (L2 mode), 0 in decoupled mode
    float wd_w;    // weight decay added to the update (decoupled mode), 0 in L2 mode
    float bc1, bc2, rbc1, rbc2;
};

__device__ __noinline__ GroupK derive_group(const ElxHyper& h, int step) {
    GroupK k;
    k.lr = h.lr;
    k.beta1 = h.beta1;
    k.beta2 = h.beta2;
    k.omb1 = 1.0f - h.beta1;
    k.omb2 = 1.0f - h.beta2;
    k.eps = h.eps;
    k.wd_l2 = h.adamw_mode ? 0.0f : h.weight_decay;
    k.wd_w = h.adamw_mode ? h.weight_decay : 0.0f;
    double bc1 = 1.0, bc2 = 1.0;
    if (h.bias_correction) {
        // 1 - beta^t evaluated in double from the fp32 betas, then rounded to fp32
        bc1 = 1.0 - pow(static_cast<double>(h.beta1), static_cast<double>(step));
        bc2 = 1.0 - pow(static_cast<double>(h.beta2), static_cast<double>(step));
    }
    k.bc1 = static_cast<float>(bc1);
    k.bc2 = static_cast<float>(bc2);
    k.rbc1 = static_cast<float>(1.0 / bc1);
    k.rbc2 = static_cast<float>(1.0 / bc2);
    return k;
}

// IEEE division and square root whose zero operands never reach the instruction sequence: __fdiv_rn and
// __fsqrt_rn handle a zero (like a denormal) on a slow path that a whole warp takes when one lane needs it, and
// states with many exact zeros -- moments of parameters that never had a gradient -- made a launch take twice as
// long (14.2 ms against 7.2 ms on an all-zero state).  For x = +-0 and y > 0 (inf included) the quotient is x itself,
// and the square root of +-0 is itself: the same bits as the plain operations, for every input.
__device__ __forceinline__ float div_or_zero(float x, float y) {
    const bool zero = x == 0.0f && y > 0.0f;
    const float q = __fdiv_rn(zero ? 1.0f : x, y);
    return zero ? x : q;
}
__device__ __forceinline__ float sqrt_or_zero(float x) {
    const bool zero = x == 0.0f;
    const float r = __fsqrt_rn(zero ? 1.0f : x);
    return zero ? x : r;
}

// How the gradient is unscaled in this launch.
enum { kNoDiv = 0, kMulInv = 1, kTrueDiv = 2 };

template <int MATH>
__device__ __forceinline__ void adam_elem(float& p, float& m, float& v, float g, const GroupK& k, int div_mode,
                                          float div, float inv_div) {
    if (div_mode == kMulInv) g *= inv_div;                    // exact: the divisor is a power of two
    else if (div_mode == kTrueDiv) g = div_or_zero(g, div);
    g = fmaf(k.wd_l2, p, g);
    m = fmaf(k.beta1, m, k.omb1 * g);
    v = fmaf(k.beta2, v, (k.omb2 * g) * g);
    float upd;
    if constexpr (MATH == 1) {
        float mhat = div_or_zero(m, k.bc1);
        float vhat = div_or_zero(v, k.bc2);
        float denom = sqrt_or_zero(vhat) + k.eps;
        upd = div_or_zero(mhat, denom);
    } else {
        float mhat = m * k.rbc1;
        float vhat = v * k.rbc2;
        float denom = __fsqrt_rn(vhat) + k.eps;
        upd = __fdividef(mhat, denom);
    }
    upd = fmaf(k.wd_w, p, upd);
    p = fmaf(-k.lr, upd, p);
}

struct AdamArgs {
    const ElxChunkDesc* descs;
    const ElxSeg* segs;
    const ElxHyper* hyper;
    ElxCtl* ctl;
    int first, count, n_groups, inline_tables;
    int64_t n_tiles;
    // push all-gather: the refreshed working copy also goes to every rank's gather block (world > 0)
    ElxPeerTable push;
    const int64_t* push_off;   // per descriptor: element offset of the chunk's block inside the slabs
    int force_direct;          // always the ld/st variant (shards in mapped host memory)
    // out-of-place update: the new master and moments of descriptor c go to shadow[c]'s arrays (bulk-copy
    // variant only); NULL = in place
    const ElxChunkDesc* shadow;
    // single-pass step over two sets of state (descs = set 0, shadow = set 1)
    int spec;                  // 1: read the set ctl->cur_set names, write the other one, probe the gradients in flight
    int repair;                // 1: run only when ctl->repair is set; rebuild the working copies from the current set
    uint32_t* chunk_flags;     // per-descriptor overflow words raised by the in-flight probe (may be null)
    // collectives through the switch: multicast addresses of all ranks' gradient / gather slabs (null = none)
    const char* mc_grads;
    char* mc_gather;
    ElxPeerTable grads;        // the gradient slabs as plain peer addresses (ragged tiles; all tiles when `pull`)
    int pull;                  // 1: the gradient of a tile is the rank average of the slabs, fetched in this kernel
    // single-shard form: the three tables travel in the kernel parameters
    ElxChunkDesc one_desc;
    ElxSeg one_seg;
    ElxHyper one_hyper;
};

// Push all-gather: element offset of this rank's shard of descriptor `c` inside every rank's gather slab.
__device__ __forceinline__ int64_t push_base_elem(const AdamArgs& a, int c, int64_t n_shard) {
    return a.push_off[c] + static_cast<int64_t>(a.push.rank) * n_shard;
}

// Skipped step: the low-precision shard holds gradients and must become parameters again.
// CTA-collective; s_cur is a shared-memory cursor that cursor_reset() has initialised.
template <int DT, int EPT>
__device__ __forceinline__ bool copyback_tiles(const AdamArgs& a, const ElxChunkDesc* __restrict__ descs,
                                               ChunkCursor& s_cur, bool active, int n_active) {
    // every thread of the CTA takes part in the chunk lookup (it synchronises the CTA); the first n_active
    // threads, those with `active` set, move the data
    bool bad_desc = false;
    const int64_t tile_lo = descs[a.first].tile_begin;
    for (int64_t it = blockIdx.x; it < a.n_tiles; it += gridDim.x) {
        const int64_t t = tile_lo + it;
        if (!locate_chunk(descs, a.first, a.count, t, s_cur) || s_cur.d.dtype != DT) {
            bad_desc = true;
            continue;
        }
        if (!active) continue;
        const int64_t e0 = (t - s_cur.t0) * kTile;
        const int64_t e1 = min(e0 + kTile, s_cur.d.n_shard);
        float* const master = s_cur.d.master;
        void* const lowp = s_cur.d.grad_param;
        const int world = a.push.world;
        const int64_t pb = world > 0 ? push_base_elem(a, s_cur.index, s_cur.d.n_shard) : 0;
        if ((e1 - e0 == kTile) && s_cur.vec_ok && (pb & 15) == 0) {
            float p[EPT];
            load_f32<EPT>(master, e0, p);
            store_lowp<DT, EPT>(lowp, e0, p);
            for (int j = 0; j < world; ++j) store_lowp<DT, EPT>(a.push.base[j], pb + e0, p);
        } else {
            typename Lp<DT>::T* out = static_cast<typename Lp<DT>::T*>(lowp);
            for (int64_t e = e0 + threadIdx.x; e < e1; e += n_active) {
                const typename Lp<DT>::T val = Lp<DT>::from_float(master[e]);
                out[e] = val;
                for (int j = 0; j < world; ++j) static_cast<typename Lp<DT>::T*>(a.push.base[j])[pb + e] = val;
            }
        }
    }
    return bad_desc;
}

template <int DT, int EPT, int MATH, int MINB>
__global__ void __launch_bounds__(kTile / EPT, MINB) adam_kernel(const __grid_constant__ AdamArgs a) {
    __shared__ GroupK s_group[kMaxGroups];
    __shared__ ChunkCursor s_cur;
    __shared__ SegCursor s_seg;

    const ElxChunkDesc* __restrict__ descs = a.inline_tables ? &a.one_desc : a.descs;
    const ElxSeg* __restrict__ segs = a.inline_tables ? &a.one_seg : a.segs;
    const ElxHyper* __restrict__ hyper = a.inline_tables ? &a.one_hyper : a.hyper;
    ElxCtl* ctl = a.ctl;

    const bool skip = ctl->skip != 0;
    const float div = ctl->div_scale;
    const float inv_div = ctl->inv_div;
    const int div_mode = div > 0.0f ? (inv_div != 0.0f ? kMulInv : kTrueDiv) : kNoDiv;

    if (!skip) {
        const int step = ctl->step;
        for (int gi = threadIdx.x; gi < a.n_groups; gi += blockDim.x) s_group[gi] = derive_group(hyper[gi], step);
    }
    if (threadIdx.x == 0) {
        s_seg.b = s_seg.e = 0;
        s_seg.group = -1;
        s_seg.chunk = -1;
    }
    cursor_reset(s_cur);

    const int64_t tile_lo = descs[a.first].tile_begin;
    float nan_acc = 0.0f;   // becomes NaN once a non-finite gradient is multiplied into it
    bool bad_desc = false;

    if (skip) {
        bad_desc = copyback_tiles<DT, EPT>(a, descs, s_cur, true, blockDim.x);
        if (__ballot_sync(0xFFFFFFFFu, bad_desc) && (threadIdx.x & 31) == 0) atomicOr(&ctl->status, ELX_STAT_BAD_DESC);
        return;
    }

    for (int64_t it = blockIdx.x; it < a.n_tiles; it += gridDim.x) {
        const int64_t t = tile_lo + it;
        if (!locate_chunk(descs, a.first, a.count, t, s_cur) || s_cur.d.dtype != DT) {
            bad_desc = true;
            continue;
        }
        const int64_t n_shard = s_cur.d.n_shard;
        const int64_t e0 = (t - s_cur.t0) * kTile;
        const int64_t e1 = min(e0 + kTile, n_shard);
        const bool full = (e1 - e0 == kTile) && s_cur.vec_ok;
        float* const master = s_cur.d.master;
        void* const lowp = s_cur.d.grad_param;
        const void* const gsrc = grad_source(s_cur.d);

        // segment that contains e0 (CTA-uniform; refreshed by one thread when e0 leaves the cached one)
        const ElxSeg* csegs = segs + s_cur.d.seg_first;
        const int n_segs = s_cur.d.seg_count;
        if (s_seg.chunk != s_cur.index || e0 < s_seg.b || e0 >= s_seg.e) {
            __syncthreads();
            if (threadIdx.x == 0) {
                const int si = find_seg(csegs, n_segs, e0);
                s_seg.chunk = s_cur.index;
                if (si >= 0) {
                    s_seg.b = csegs[si].begin;
                    s_seg.e = csegs[si].end;
                    s_seg.group = csegs[si].group;
                } else {
                    s_seg.b = s_seg.e = 0;
                    s_seg.group = -1;
                }
            }
            __syncthreads();
        }
        const int grp = s_seg.group;
        const bool one_group = s_seg.b <= e0 && e1 <= s_seg.e && grp >= 0 && grp < a.n_groups;
        float* const exp_avg = s_cur.d.exp_avg;
        float* const exp_avg_sq = s_cur.d.exp_avg_sq;

        if (full && one_group) {
            const GroupK k = s_group[grp];
            float g[EPT], p[EPT], m[EPT], v[EPT];
            load_lowp<DT, EPT>(gsrc, e0, g);
            load_f32<EPT>(master, e0, p);
            load_f32<EPT>(exp_avg, e0, m);
            load_f32<EPT>(exp_avg_sq, e0, v);
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                nan_acc = fmaf(0.0f, g[j], nan_acc);
                adam_elem<MATH>(p[j], m[j], v[j], g[j], k, div_mode, div, inv_div);
            }
            store_f32<EPT>(master, e0, p);
            store_f32<EPT>(exp_avg, e0, m);
            store_f32<EPT>(exp_avg_sq, e0, v);
            store_lowp<DT, EPT>(lowp, e0, p);
        } else if (full && e0 >= s_cur.d.n_valid) {
            // padding past valid_end: no segment reaches it, only the working copy is refreshed
            float p[EPT];
            load_f32<EPT>(master, e0, p);
            store_lowp<DT, EPT>(lowp, e0, p);
        } else {
            // ragged tile: shard tail, segment boundary, uncovered elements or unaligned pointers
            typename Lp<DT>::T* gp = static_cast<typename Lp<DT>::T*>(lowp);
            const typename Lp<DT>::T* gin = static_cast<const typename Lp<DT>::T*>(gsrc);
            for (int64_t e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
                float p = master[e];
                const int si = find_seg(csegs, n_segs, e);
                if (si >= 0 && e < csegs[si].end) {
                    const int ge = csegs[si].group;
                    if (ge >= 0 && ge < a.n_groups) {
                        const GroupK k = s_group[ge];
                        float g = Lp<DT>::to_float(gin[e]);
                        float m = exp_avg[e], v = exp_avg_sq[e];
                        nan_acc = fmaf(0.0f, g, nan_acc);
                        adam_elem<MATH>(p, m, v, g, k, div_mode, div, inv_div);
                        master[e] = p;
                        exp_avg[e] = m;
                        exp_avg_sq[e] = v;
                    }
                }
                gp[e] = Lp<DT>::from_float(p);
            }
        }
    }

    // warp-reduced report of a non-finite gradient met on an applied step
    const bool late = nan_acc != nan_acc;
    const unsigned ballot = __ballot_sync(0xFFFFFFFFu, late);
    const unsigned ballot_desc = __ballot_sync(0xFFFFFFFFu, bad_desc);
    if ((threadIdx.x & 31) == 0) {
        if (ballot) {
            atomicOr(&ctl->late_inf, 1u);
            atomicOr(&ctl->status, ELX_STAT_LATE_INF);
        }
        if (ballot_desc) atomicOr(&ctl->status, ELX_STAT_BAD_DESC);
    }
}

// ------------------------------------------------------------------------------------------------
// Adam, bulk-copy pipelined variant
// ------------------------------------------------------------------------------------------------
//
// Same arithmetic, different data movement: whole tiles stream between HBM and shared memory with
// cp.async.bulk (the TMA unit's untiled form), completion tracked by mbarriers, so loads of the next tiles
// and stores of the previous one are in flight while the CTA's warps compute on the current one out of
// shared memory.  One CTA per SM: 16 computing warps plus one warp whose first lane -- the data mover --
// issues every bulk copy; a ring of S stages of one tile each (16-bit gradients: 8 KB + 3 x 16 KB = 56 KB
// per stage; S = 4 where that fits, else 3).
//
//   computing warps, tile k (stage s = k % S):
//       wait full[s]; read g,p,m,v from the stage; update; write p,m,v,p16 back in place;
//       fence.proxy.async; barrier among the computing warps; one arrival on done[s]
//   data mover, tile k:
//       wait done[s]; 4 bulk stores stage s -> HBM, commit; wait until the stores of tile k-1 have read
//       their stage; classify tile k+S-1, publish its slot, arm full[(k+S-1) % S], issue its 4 bulk loads
//
// The mover's bookkeeping (tile classification, descriptor and segment lookup, some hundred instructions per
// tile) used to be done by thread 0 between two CTA-wide barriers, i.e. on every warp's path.  Measured on the
// GPT-2-XL chunk set, same GPU, back to back: 7.17 ms per launch with thread 0 as the mover, 6.98 ms with the
// warp of its own; before that, three stages against four: 7.13 ms against 6.97 ms.
//
// Ragged tiles (shard tail, segment boundary, unaligned pointers) bypass the pipeline and are updated
// in place in global memory by the same scalar path as the direct kernel.  Every mbarrier wait is
// bounded: on expiry the CTA raises ELX_STAT_TIMEOUT, stops issuing copies, drains and returns.

constexpr int kTmaThreads = 512;                   // the warps that compute
constexpr int kTmaBlock = kTmaThreads + 32;        // plus one warp whose first lane moves the data

// Stages of the ring.  Three everywhere, except the default instantiations (16-bit chunks, IEEE arithmetic, no
// peers' slices beside the stage): four 56 KB stages plus the kernel's static shared memory just fit into the
// 227 KB a CTA may have, provided the per-group constants are kept in their compact form (below).
template <int DT, int MATH, int PW>
struct TmaRing {
    static constexpr int kStages = (DT != ELX_F32 && MATH == 1 && PW <= 1) ? 4 : 3;
};

// The constants of a parameter group as the four-stage instantiations keep them in shared memory (32 bytes
// instead of 48): what IEEE mode needs; 1 - beta is recomputed where it is used (the same single operation).
struct GroupCompact {
    float lr, beta1, beta2, eps, wd_l2, wd_w, bc1, bc2;
};
__device__ __forceinline__ GroupCompact pack_group(const GroupK& k) {
    return GroupCompact{k.lr, k.beta1, k.beta2, k.eps, k.wd_l2, k.wd_w, k.bc1, k.bc2};
}
__device__ __forceinline__ GroupCompact pack_group(const GroupCompact& k) { return k; }
__device__ __forceinline__ GroupK unpack_group(const GroupK& k) { return k; }
__device__ __forceinline__ GroupK unpack_group(const GroupCompact& c) {
    GroupK k;
    k.lr = c.lr;
    k.beta1 = c.beta1;
    k.omb1 = 1.0f - c.beta1;
    k.beta2 = c.beta2;
    k.omb2 = 1.0f - c.beta2;
    k.eps = c.eps;
    k.wd_l2 = c.wd_l2;
    k.wd_w = c.wd_w;
    k.bc1 = c.bc1;
    k.bc2 = c.bc2;
    k.rbc1 = 0.0f;   // reciprocal-multiply mode never runs with the compact form
    k.rbc2 = 0.0f;
    return k;
}

// kTileRefresh: a whole tile that no segment covers (the padding past valid_end, a gap between segments):
// only its master goes through the pipeline and only the working copy comes back (6 bytes per element)
enum { kTileNone = 0, kTileBulk = 1, kTileRagged = 2, kTileBad = 3, kTileRefresh = 4 };

// What the producer thread decided about one tile, published to the CTA through shared memory.
struct TileSlot {
    float* master;
    float* exp_avg;
    float* exp_avg_sq;
    float* out_master;      // where the updated values go: the same arrays, or the other set's
    float* out_exp_avg;
    float* out_exp_avg_sq;
    void* lowp;
    const void* gsrc;       // where the gradient is read: the low-precision shard itself or a separate source
    const ElxSeg* segs;
    int64_t e0, e1;
    int64_t n_valid;
    int64_t push_elem;   // element offset of this tile inside every rank's gather (and gradient) slab
    int n_segs;
    int group;
    int kind;
    int chunk;
};

template <int DT>
struct TmaStage {
    static constexpr int kLowpBytes = kTile * Lp<DT>::kBytes;
    static constexpr int kF32Bytes = kTile * 4;
    static constexpr int kBytes = kLowpBytes + 3 * kF32Bytes;
};

// Producer-side (one thread) chunk and segment lookup with its own register cursors.
struct ProducerCursor {
    int64_t t0 = 0, t1 = 0;
    int index = -1;
    bool vec_ok = false;
    ElxChunkDesc d;
    float* out_master = nullptr;
    float* out_exp_avg = nullptr;
    float* out_exp_avg_sq = nullptr;
    bool shadow_ok = true;
    int64_t seg_b = 0, seg_e = 0;
    int seg_group = -1;
    int seg_chunk = -1;
};

// src: the table whose master and moments are read.  dst: the table whose arrays receive the update, or
// null for an update in place.  probe_gaps: whole tiles below valid_end that no segment covers still have
// their gradients looked at (single-pass step), so they are not refresh-only.
template <int DT>
__device__ __forceinline__ void classify_tile(const AdamArgs& a, const ElxChunkDesc* __restrict__ src,
                                              const ElxChunkDesc* __restrict__ dst, const ElxSeg* __restrict__ segs,
                                              bool probe_gaps, int64_t t, ProducerCursor& pc, TileSlot& out) {
    if (!(t >= pc.t0 && t < pc.t1)) {
        int lo = a.first, hi = a.first + a.count - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (src[mid].tile_begin <= t) lo = mid; else hi = mid - 1;
        }
        pc.d = src[lo];
        pc.index = lo;
        pc.t0 = pc.d.tile_begin;
        pc.t1 = pc.t0 + tiles_of(pc.d.n_shard);
        uintptr_t bits = reinterpret_cast<uintptr_t>(pc.d.master) | reinterpret_cast<uintptr_t>(pc.d.exp_avg) |
                         reinterpret_cast<uintptr_t>(pc.d.exp_avg_sq) | reinterpret_cast<uintptr_t>(pc.d.grad_param) |
                         reinterpret_cast<uintptr_t>(pc.d.grad_src);
        pc.out_master = pc.d.master;
        pc.out_exp_avg = pc.d.exp_avg;
        pc.out_exp_avg_sq = pc.d.exp_avg_sq;
        pc.shadow_ok = true;
        if (dst) {
            const ElxChunkDesc sd = dst[lo];
            pc.out_master = sd.master;
            pc.out_exp_avg = sd.exp_avg;
            pc.out_exp_avg_sq = sd.exp_avg_sq;
            // the other descriptor must describe the same shard, with arrays of its own
            pc.shadow_ok = sd.n_shard == pc.d.n_shard && sd.tile_begin == pc.d.tile_begin && sd.master &&
                           sd.exp_avg && sd.exp_avg_sq;
            bits |= reinterpret_cast<uintptr_t>(sd.master) | reinterpret_cast<uintptr_t>(sd.exp_avg) |
                    reinterpret_cast<uintptr_t>(sd.exp_avg_sq);
        }
        pc.vec_ok = (bits & 31u) == 0;
    }
    if (!(t >= pc.t0 && t < pc.t1) || pc.d.dtype != DT || !pc.shadow_ok) {
        out.kind = kTileBad;
        return;
    }
    const int64_t e0 = (t - pc.t0) * kTile;
    const int64_t e1 = min(e0 + kTile, pc.d.n_shard);
    const ElxSeg* csegs = segs + pc.d.seg_first;
    if (pc.seg_chunk != pc.index || e0 < pc.seg_b || e0 >= pc.seg_e) {
        pc.seg_chunk = pc.index;
        const int si = find_seg(csegs, pc.d.seg_count, e0);
        if (si >= 0) {
            pc.seg_b = csegs[si].begin;
            pc.seg_e = csegs[si].end;
            pc.seg_group = csegs[si].group;
        } else {
            pc.seg_b = pc.seg_e = 0;
            pc.seg_group = -1;
        }
    }
    const bool one_group = pc.seg_b <= e0 && e1 <= pc.seg_e && pc.seg_group >= 0 && pc.seg_group < a.n_groups;
    out.master = pc.d.master;
    out.exp_avg = pc.d.exp_avg;
    out.exp_avg_sq = pc.d.exp_avg_sq;
    out.out_master = pc.out_master;
    out.out_exp_avg = pc.out_exp_avg;
    out.out_exp_avg_sq = pc.out_exp_avg_sq;
    out.lowp = pc.d.grad_param;
    out.gsrc = grad_source(pc.d);
    out.segs = csegs;
    out.n_segs = pc.d.seg_count;
    out.e0 = e0;
    out.e1 = e1;
    out.n_valid = pc.d.n_valid;
    out.group = pc.seg_group;
    out.chunk = pc.index;
    out.push_elem = a.push.world > 0 ? push_base_elem(a, pc.index, pc.d.n_shard) + e0 : 0;
    const bool push_ok = a.push.world == 0 || (out.push_elem & 15) == 0;   // bulk copies need 16-byte alignment
    const bool whole = e1 - e0 == kTile && pc.vec_ok && push_ok;
    if (whole && one_group) out.kind = kTileBulk;
    else if (whole && (e0 >= pc.d.n_valid || (!probe_gaps && range_uncovered(csegs, pc.d.seg_count, e0, e1, pc.d.n_valid))))
        out.kind = kTileRefresh;
    else out.kind = kTileRagged;
}

// multimem: one access for all ranks of an NVLink domain, carried out by the switch.  ld_reduce returns the
// sum over the ranks' copies of the addressed words (fp32 accumulation, one rounding to the 16-bit format);
// st delivers the words to every rank's copy.  8 bytes (4 elements) per access.
template <int DT>
__device__ __forceinline__ uint2 mm_ld_reduce8(const void* mc) {
    uint2 r;
    if constexpr (DT == ELX_BF16) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.bf16x2 {%0,%1}, [%2];"
                     : "=r"(r.x), "=r"(r.y) : "l"(mc) : "memory");
    } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v2.f16x2 {%0,%1}, [%2];"
                     : "=r"(r.x), "=r"(r.y) : "l"(mc) : "memory");
    }
    return r;
}
template <int DT>
__device__ __forceinline__ uint32_t mm_ld_reduce4(const void* mc) {
    uint32_t r;
    if constexpr (DT == ELX_BF16) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.bf16x2 %0, [%1];" : "=r"(r) : "l"(mc) : "memory");
    } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.f16x2 %0, [%1];" : "=r"(r) : "l"(mc) : "memory");
    }
    return r;
}
__device__ __forceinline__ void mm_st8(void* mc, uint2 v) {
    asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
}

// MM: the gradient tile is the switch-side sum over all ranks' gradient slabs and the refreshed working copy
// is multicast to all ranks' gather slabs (16-bit chunks only).
// PW > 1: the gradient tile is the rank average of PW ranks' gradient slabs, fetched here with PW plain
// (non-multicast) bulk loads per tile -- the own slice into the stage's low-precision slot, the peers' slices
// into PW - 1 staging slots behind the stage -- and summed by the threads exactly as the pull kernel sums
// (fp32, rank order, one rounding to the chunk dtype).  16-bit chunks; shared memory allows PW = 2.
template <int DT, int MATH, bool MM, int PW, int STAGES>
__global__ void __launch_bounds__(kTmaBlock, 1) adam_tma_kernel(const __grid_constant__ AdamArgs a) {
    using Stage = TmaStage<DT>;
    static_assert(!MM || DT != ELX_F32, "the multicast form is for 16-bit chunks");
    static_assert(PW == 0 || (PW > 1 && !MM && DT != ELX_F32), "the pulling form is for 16-bit chunks, without multicast");
    constexpr int kPeerSlots = PW > 1 ? PW - 1 : 0;
    constexpr int kStageBytes = Stage::kBytes + kPeerSlots * Stage::kLowpBytes;
    constexpr int kTmaStages = STAGES;
    static_assert(STAGES == 3 || STAGES == TmaRing<DT, MATH, PW>::kStages, "a ring this deep does not fit");
    using GroupStore = typename std::conditional<kTmaStages == 4, GroupCompact, GroupK>::type;
    extern __shared__ __align__(128) unsigned char s_dyn[];
    __shared__ GroupStore s_group[kMaxGroups];
    __shared__ TileSlot s_slot[kTmaStages];
    // the ring plus everything static has to fit the 227 KB a CTA may have (the four-stage ring leaves 3 KB)
    static_assert(kTmaStages * kStageBytes + sizeof(GroupStore) * kMaxGroups + sizeof(TileSlot) * kTmaStages +
                          2 * sizeof(uint64_t) * kTmaStages + 64 <= 227 * 1024,
                  "ring and static shared memory exceed a CTA's shared memory");
    __shared__ __align__(8) uint64_t s_full[kTmaStages];   // the loads of a stage have landed (and its slot is published)
    __shared__ __align__(8) uint64_t s_done[kTmaStages];   // the computing warps are through with a stage
    __shared__ int s_abort;

    const bool mover = threadIdx.x == kTmaThreads;         // the one thread that issues every bulk copy
    const bool computes = threadIdx.x < kTmaThreads;
    const ElxChunkDesc* __restrict__ descs = a.inline_tables ? &a.one_desc : a.descs;
    const ElxSeg* __restrict__ segs = a.inline_tables ? &a.one_seg : a.segs;
    const ElxHyper* __restrict__ hyper = a.inline_tables ? &a.one_hyper : a.hyper;
    ElxCtl* ctl = a.ctl;

    // which table is read and which is written: in place, out of place (shadow), or the two sets of the
    // single-pass step whose roles follow ctl->cur_set
    const bool spec = a.spec != 0;
    const bool flipped = spec && ctl->cur_set != 0;
    const ElxChunkDesc* __restrict__ src = flipped ? a.shadow : descs;
    const ElxChunkDesc* __restrict__ dst = spec ? (flipped ? descs : a.shadow) : a.shadow;

    if (a.repair && ctl->repair == 0) return;
    if (ctl->skip != 0 || a.repair) {
        // skipped step: copy-back only, with direct accesses (6 bytes per element, no staging needed)
        // the ring is not used on this path: the cursor lives at its start
        ChunkCursor& s_cur = *reinterpret_cast<ChunkCursor*>(s_dyn);
        cursor_reset(s_cur);
        const bool bad = copyback_tiles<DT, kTile / kTmaThreads>(a, src, s_cur, computes, kTmaThreads);
        if (__ballot_sync(0xFFFFFFFFu, bad) && (threadIdx.x & 31) == 0) atomicOr(&ctl->status, ELX_STAT_BAD_DESC);
        return;
    }

    const float div = ctl->div_scale;
    const float inv_div = ctl->inv_div;
    const int div_mode = div > 0.0f ? (inv_div != 0.0f ? kMulInv : kTrueDiv) : kNoDiv;
    const int step = ctl->step;
    for (int gi = threadIdx.x; gi < a.n_groups; gi += blockDim.x) {
        const GroupK derived = derive_group(hyper[gi], step);
        if constexpr (kTmaStages == 4) s_group[gi] = pack_group(derived);
        else s_group[gi] = derived;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTmaStages; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_done[s], 1);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t tile_lo = src[a.first].tile_begin;
    const int64_t my_tiles = blockIdx.x < a.n_tiles ? (a.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const float inv_w = (MM || PW > 1) ? 1.0f / static_cast<float>(a.push.world) : 1.0f;
    // MM: no gradient tile from HBM; PW: the peers' slices come in beside the stage
    constexpr uint32_t kLoadBytes = MM ? 3 * Stage::kF32Bytes : kStageBytes;
    ProducerCursor pc;
    float nan_acc = 0.0f;
    bool bad_desc = false;

    // producer: classify tile k of this CTA, publish it in its stage's slot, start its loads
    auto produce = [&](int64_t k) {
        const int s = static_cast<int>(k % kTmaStages);
        TileSlot slot;
        slot.kind = kTileNone;
        classify_tile<DT>(a, src, dst, segs, spec, tile_lo + blockIdx.x + k * gridDim.x, pc, slot);
        s_slot[s] = slot;
        if (slot.kind == kTileBulk) {
            unsigned char* base = s_dyn + static_cast<size_t>(s) * kStageBytes;
            mbar_arrive_expect_tx(&s_full[s], kLoadBytes);
            if constexpr (PW > 1) {
                // slice of every rank's gradient block that belongs to this tile: the own one into the stage's
                // low-precision slot, the others (over NVLink) into the slots behind the stage
#pragma unroll
                for (int i = 0; i < PW; ++i) {
                    const int j = (a.grads.rank + i) % PW;
                    unsigned char* dst = i == 0 ? base : base + Stage::kBytes + (i - 1) * Stage::kLowpBytes;
                    bulk_g2s(dst, static_cast<const char*>(a.grads.base[j]) + slot.push_elem * Lp<DT>::kBytes,
                             Stage::kLowpBytes, &s_full[s]);
                }
            } else if (!MM) {
                bulk_g2s(base, static_cast<const char*>(slot.gsrc) + slot.e0 * Lp<DT>::kBytes, Stage::kLowpBytes,
                         &s_full[s]);
            }
            bulk_g2s(base + Stage::kLowpBytes, slot.master + slot.e0, Stage::kF32Bytes, &s_full[s]);
            bulk_g2s(base + Stage::kLowpBytes + Stage::kF32Bytes, slot.exp_avg + slot.e0, Stage::kF32Bytes, &s_full[s]);
            bulk_g2s(base + Stage::kLowpBytes + 2 * Stage::kF32Bytes, slot.exp_avg_sq + slot.e0, Stage::kF32Bytes,
                     &s_full[s]);
        } else if (slot.kind == kTileRefresh) {
            unsigned char* base = s_dyn + static_cast<size_t>(s) * kStageBytes;
            mbar_arrive_expect_tx(&s_full[s], Stage::kF32Bytes);
            bulk_g2s(base + Stage::kLowpBytes, slot.master + slot.e0, Stage::kF32Bytes, &s_full[s]);
        } else {
            mbar_arrive(&s_full[s]);   // nothing to load: the phase completes at once and publishes the slot
        }
    };

    if (mover) {
        for (int64_t k = 0; k < my_tiles && k < kTmaStages - 1; ++k) produce(k);
    }

    // MM: the thread's own 2 x 4 gradient elements of the NEXT tile, asked from the switch one tile ahead and
    // held in registers (a thread consumes exactly the elements it fetched)
    constexpr int kHalves = kTile / (kTmaThreads * 4);   // 2
    uint2 g_now[kHalves], g_next[kHalves];
    auto fetch = [&](int64_t k, uint2 (&g)[kHalves]) {
        if (k >= my_tiles) return;
        const TileSlot& nx = s_slot[k % kTmaStages];
        if (nx.kind != kTileBulk) return;
#pragma unroll
        for (int h = 0; h < kHalves; ++h) {
            const int e = h * (kTmaThreads * 4) + threadIdx.x * 4;
            g[h] = mm_ld_reduce8<DT == ELX_F32 ? ELX_F16 : DT>(a.mc_grads + (nx.push_elem + e) * 2);
        }
    };
    if constexpr (MM) {
        __syncthreads();   // the first slots are published
        if (computes) fetch(0, g_now);
    }

    // barrier of the computing warps alone (the data mover runs on its own clock)
    auto sync_computing = [] { asm volatile("bar.sync 1, %0;" ::"n"(kTmaThreads) : "memory"); };

    int64_t k = 0;
    if (computes) {
    for (; k < my_tiles; ++k) {
        const int s = static_cast<int>(k % kTmaStages);
        const uint32_t parity = static_cast<uint32_t>((k / kTmaStages) & 1);
        if (!mbar_wait_bounded(&s_full[s], parity)) s_abort = 1;
        sync_computing();
        if (s_abort) break;
        const TileSlot slot = s_slot[s];   // into registers: measured 1.3 % faster than reading the fields from shared memory
        unsigned char* base = s_dyn + static_cast<size_t>(s) * kStageBytes;
        if constexpr (MM) {
            // the slot of tile k + 1 is published once its loads have been started; they were started three tiles ago
            if (k + 1 < my_tiles) {
                const int s1 = static_cast<int>((k + 1) % kTmaStages);
                if (mbar_wait_bounded(&s_full[s1], static_cast<uint32_t>(((k + 1) / kTmaStages) & 1))) fetch(k + 1, g_next);
                else s_abort = 1;   // seen by every thread at the next tile's barrier
            }
        }

        if (slot.kind == kTileBulk) {
            const GroupK k_ = unpack_group(s_group[slot.group]);
            float* sp = reinterpret_cast<float*>(base + Stage::kLowpBytes);
            float* sm = sp + kTile;
            float* sv = sm + kTile;
            // a thread owns 2 x 4 consecutive elements, 2048 apart: conflict-free 128-bit shared accesses
#pragma unroll
            for (int h = 0; h < kHalves; ++h) {
                const int e = h * (kTmaThreads * 4) + threadIdx.x * 4;
                float4 p = *reinterpret_cast<float4*>(sp + e);
                float4 m = *reinterpret_cast<float4*>(sm + e);
                float4 v = *reinterpret_cast<float4*>(sv + e);
                float g[4];
                if constexpr (DT == ELX_F32) {
                    const float4 gg = *reinterpret_cast<const float4*>(base + static_cast<size_t>(e) * 4);
                    g[0] = gg.x; g[1] = gg.y; g[2] = gg.z; g[3] = gg.w;
                } else {
                    if constexpr (PW > 1) {
                        // rank average as the pull kernel forms it: fp32, rank order, rounded once to the chunk dtype
                        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int j = 0; j < PW; ++j) {
                            const int i = (j - a.grads.rank + PW) % PW;   // which slot holds rank j's slice
                            const unsigned char* slice = i == 0 ? base : base + Stage::kBytes + (i - 1) * Stage::kLowpBytes;
                            const uint2 w = *reinterpret_cast<const uint2*>(slice + static_cast<size_t>(e) * 2);
                            const float2 a0 = Lp<DT>::unpack2(w.x), a1 = Lp<DT>::unpack2(w.y);
                            acc[0] = fmaf(a0.x, inv_w, acc[0]);
                            acc[1] = fmaf(a0.y, inv_w, acc[1]);
                            acc[2] = fmaf(a1.x, inv_w, acc[2]);
                            acc[3] = fmaf(a1.y, inv_w, acc[3]);
                        }
                        const float2 r0 = Lp<DT>::unpack2(Lp<DT>::pack2(acc[0], acc[1]));
                        const float2 r1 = Lp<DT>::unpack2(Lp<DT>::pack2(acc[2], acc[3]));
                        g[0] = r0.x; g[1] = r0.y; g[2] = r1.x; g[3] = r1.y;
                    } else {
                        uint2 gg;
                        if constexpr (MM) gg = g_now[h];
                        else gg = *reinterpret_cast<const uint2*>(base + static_cast<size_t>(e) * 2);
                        const float2 a0 = Lp<DT>::unpack2(gg.x), a1 = Lp<DT>::unpack2(gg.y);
                        g[0] = a0.x; g[1] = a0.y; g[2] = a1.x; g[3] = a1.y;
                        if constexpr (MM) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) g[j] *= inv_w;   // the switch summed; the step wants the average
                        }
                    }
                }
                float pp[4] = {p.x, p.y, p.z, p.w}, mm[4] = {m.x, m.y, m.z, m.w}, vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    nan_acc = fmaf(0.0f, g[j], nan_acc);
                    adam_elem<MATH>(pp[j], mm[j], vv[j], g[j], k_, div_mode, div, inv_div);
                }
                *reinterpret_cast<float4*>(sp + e) = make_float4(pp[0], pp[1], pp[2], pp[3]);
                *reinterpret_cast<float4*>(sm + e) = make_float4(mm[0], mm[1], mm[2], mm[3]);
                *reinterpret_cast<float4*>(sv + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
                if constexpr (DT == ELX_F32) {
                    *reinterpret_cast<float4*>(base + static_cast<size_t>(e) * 4) = make_float4(pp[0], pp[1], pp[2], pp[3]);
                } else {
                    uint2 out;
                    out.x = Lp<DT>::pack2(pp[0], pp[1]);
                    out.y = Lp<DT>::pack2(pp[2], pp[3]);
                    *reinterpret_cast<uint2*>(base + static_cast<size_t>(e) * 2) = out;
                    // all-gather: one store to the multicast address reaches every rank's gather block
                    if constexpr (MM) mm_st8(a.mc_gather + (slot.push_elem + e) * 2, out);
                }
            }
            fence_async_smem();   // the bulk stores below read what the threads just wrote
        } else if (slot.kind == kTileRefresh) {
            const float* sp = reinterpret_cast<const float*>(base + Stage::kLowpBytes);
#pragma unroll
            for (int h = 0; h < kHalves; ++h) {
                const int e = h * (kTmaThreads * 4) + threadIdx.x * 4;
                const float4 p = *reinterpret_cast<const float4*>(sp + e);
                if constexpr (DT == ELX_F32) {
                    *reinterpret_cast<float4*>(base + static_cast<size_t>(e) * 4) = p;
                } else {
                    uint2 out;
                    out.x = Lp<DT>::pack2(p.x, p.y);
                    out.y = Lp<DT>::pack2(p.z, p.w);
                    *reinterpret_cast<uint2*>(base + static_cast<size_t>(e) * 2) = out;
                    if constexpr (MM) mm_st8(a.mc_gather + (slot.push_elem + e) * 2, out);
                }
            }
            fence_async_smem();
        } else if (slot.kind == kTileRagged) {
            typename Lp<DT>::T* gp = static_cast<typename Lp<DT>::T*>(slot.lowp);
            const typename Lp<DT>::T* gin = static_cast<const typename Lp<DT>::T*>(slot.gsrc);
            for (int64_t e = slot.e0 + threadIdx.x; e < slot.e1; e += kTmaThreads) {
                float p = slot.master[e];
                float g = 0.0f;
                if (e < slot.n_valid) {
                    if constexpr (MM) {
                        // the switch's own sum here too (its arithmetic is not the rank-order fp32 sum rounded once):
                        // the aligned pair that holds the element, one of its halves
                        const int64_t idx = slot.push_elem + (e - slot.e0);
                        const uint32_t pair = mm_ld_reduce4<DT>(a.mc_grads + (idx & ~static_cast<int64_t>(1)) * 2);
                        const float2 both = Lp<DT>::unpack2(pair);
                        g = ((idx & 1) ? both.y : both.x) * inv_w;
                    } else if constexpr (PW > 1) {
                        float acc = 0.0f;
                        for (int j = 0; j < PW; ++j)
                            acc = fmaf(Lp<DT>::to_float(static_cast<const typename Lp<DT>::T*>(
                                           a.grads.base[j])[slot.push_elem + (e - slot.e0)]),
                                       inv_w, acc);
                        g = Lp<DT>::to_float(Lp<DT>::from_float(acc));
                    } else {
                        g = Lp<DT>::to_float(gin[e]);
                    }
                    if (spec) nan_acc = fmaf(0.0f, g, nan_acc);   // the single-pass step probes all of [0, n_valid)
                }
                const int si = find_seg(slot.segs, slot.n_segs, e);
                if (si >= 0 && e < slot.segs[si].end) {
                    const int ge = slot.segs[si].group;
                    if (ge >= 0 && ge < a.n_groups) {
                        const GroupK k_ = unpack_group(s_group[ge]);
                        float m = slot.exp_avg[e], v = slot.exp_avg_sq[e];
                        nan_acc = fmaf(0.0f, g, nan_acc);
                        adam_elem<MATH>(p, m, v, g, k_, div_mode, div, inv_div);
                        slot.out_master[e] = p;
                        slot.out_exp_avg[e] = m;
                        slot.out_exp_avg_sq[e] = v;
                    }
                }
                const typename Lp<DT>::T val = Lp<DT>::from_float(p);
                gp[e] = val;
                for (int j = 0; j < a.push.world; ++j)
                    static_cast<typename Lp<DT>::T*>(a.push.base[j])[slot.push_elem + (e - slot.e0)] = val;
            }
        } else if (slot.kind == kTileBad) {
            bad_desc = true;
        }
        if (spec) {
            // single-pass step: a non-finite gradient met in this tile raises the overflow words now
            // (the update went to the other set and will not be adopted)
            const unsigned hit = __ballot_sync(0xFFFFFFFFu, nan_acc != nan_acc);
            if (hit && (threadIdx.x & 31) == 0) {
                atomicOr(&ctl->found_inf, 1u);
                if (a.chunk_flags) atomicOr(&a.chunk_flags[slot.chunk], 1u);
            }
            nan_acc = 0.0f;
        }
        sync_computing();   // the stage is fully written (bulk) / fully consumed
        if (threadIdx.x == 0) mbar_arrive(&s_done[s]);   // over to the data mover
        if constexpr (MM) {
#pragma unroll
            for (int h = 0; h < kHalves; ++h) g_now[h] = g_next[h];
        }
    }
    } else if (mover) {
        // The data mover: for every tile, once the computing warps are through with its stage, the bulk stores
        // of the stage and -- as soon as the stores of the tile before have read their stage -- the loads of the
        // tile that will use that stage next.  None of this is on the computing warps' path.
        for (; k < my_tiles; ++k) {
            const int s = static_cast<int>(k % kTmaStages);
            const uint32_t parity = static_cast<uint32_t>((k / kTmaStages) & 1);
            bool handed_over = false;
            for (uint32_t i = 0; i < kTmaSpinLimit && !handed_over; ++i) {
                handed_over = mbar_try_wait(&s_done[s], parity);
                if (!handed_over && *reinterpret_cast<volatile int*>(&s_abort)) break;   // the computing warps gave up
            }
            if (!handed_over) {
                s_abort = 1;
                break;
            }
            const TileSlot slot = s_slot[s];
            unsigned char* base = s_dyn + static_cast<size_t>(s) * kStageBytes;
            if (slot.kind == kTileBulk || slot.kind == kTileRefresh) {
                bulk_s2g(static_cast<char*>(slot.lowp) + slot.e0 * Lp<DT>::kBytes, base, Stage::kLowpBytes);
                if (slot.kind == kTileBulk) {
                    bulk_s2g(slot.out_master + slot.e0, base + Stage::kLowpBytes, Stage::kF32Bytes);
                    bulk_s2g(slot.out_exp_avg + slot.e0, base + Stage::kLowpBytes + Stage::kF32Bytes, Stage::kF32Bytes);
                    bulk_s2g(slot.out_exp_avg_sq + slot.e0, base + Stage::kLowpBytes + 2 * Stage::kF32Bytes,
                             Stage::kF32Bytes);
                }
                if constexpr (!MM) {
                    // push all-gather: the same 8 KB of refreshed parameters to every rank's gather block,
                    // plain (non-multicast) bulk stores, W - 1 of them crossing NVLink
                    // (start with a different rank in every CTA, so that the stores spread over all links at once)
                    for (int i = 0; i < a.push.world; ++i) {
                        const int j = (a.push.rank + 1 + i + static_cast<int>(blockIdx.x)) % a.push.world;
                        bulk_s2g(static_cast<char*>(a.push.base[j]) + slot.push_elem * Lp<DT>::kBytes, base,
                                 Stage::kLowpBytes);
                    }
                }
            }
            bulk_commit();
            if (k + kTmaStages - 1 < my_tiles) {
                bulk_wait_read<1>();   // the stage of tile k-1 has been read out by its stores
                produce(k + kTmaStages - 1);
            }
        }
        if (s_abort) {
            // gave up on tile k: the loads already issued for the tiles after it still target this CTA's
            // shared memory, so wait (bounded again) for them before the CTA may exit
            for (int64_t j = k; j < my_tiles && j < k + kTmaStages - 1; ++j)
                (void)mbar_wait_bounded(&s_full[j % kTmaStages], static_cast<uint32_t>((j / kTmaStages) & 1));
            atomicOr(&ctl->status, ELX_STAT_TIMEOUT);
        }
        bulk_wait_all();
    }

    const bool late = !spec && nan_acc != nan_acc;
    const unsigned ballot = __ballot_sync(0xFFFFFFFFu, late);
    const unsigned ballot_desc = __ballot_sync(0xFFFFFFFFu, bad_desc);
    if ((threadIdx.x & 31) == 0) {
        if (ballot) {
            atomicOr(&ctl->late_inf, 1u);
            atomicOr(&ctl->status, ELX_STAT_LATE_INF);
        }
        if (ballot_desc) atomicOr(&ctl->status, ELX_STAT_BAD_DESC);
    }
}


template <int DT>
__global__ void __launch_bounds__(256) cast_kernel(const float* __restrict__ src, void* dst, int64_t n, int vec_ok) {
    constexpr int EPT = 16;
    const int64_t n_full = vec_ok ? n / kTile : 0;
    for (int64_t t = blockIdx.x; t < n_full; t += gridDim.x) {
        float p[EPT];
        load_f32<EPT>(src, t * kTile, p);
        store_lowp<DT, EPT>(dst, t * kTile, p);
    }
    typename Lp<DT>::T* out = static_cast<typename Lp<DT>::T*>(dst);
    for (int64_t e = n_full * kTile + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < n;
         e += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[e] = Lp<DT>::from_float(src[e]);
}

template <int DT, int EPT, int MATH, int MINB>
int launch_adam_inst(const AdamArgs& a, cudaStream_t s) {
    constexpr int threads = kTile / EPT;
    static const int resident = resident_ctas(adam_kernel<DT, EPT, MATH, MINB>, threads);
    const int grid = grid_for(a.n_tiles, capped(resident, g_tune.adam_ctas_per_sm));
    if (grid < 0) return grid;
    adam_kernel<DT, EPT, MATH, MINB><<<grid, threads, 0, s>>>(a);
    return record_cuda(cudaGetLastError());
}

template <int DT, int EPT, int MATH>
int launch_adam_minb(const AdamArgs& a, cudaStream_t s) {
    return launch_adam_inst<DT, EPT, MATH, 2>(a, s);
}

template <int DT, int MATH, bool MM, int PW, int STAGES>
int launch_adam_tma_ring(const AdamArgs& a, cudaStream_t s) {
    constexpr int smem = STAGES * (TmaStage<DT>::kBytes + (PW > 1 ? (PW - 1) * TmaStage<DT>::kLowpBytes : 0));
    // the opt-in to more than 48 KB of dynamic shared memory is per device: once for each ordinal
    static bool opted_in[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    if (!opted_in[dev]) {
        const cudaError_t attr = cudaFuncSetAttribute(adam_tma_kernel<DT, MATH, MM, PW, STAGES>,
                                                      cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (attr != cudaSuccess) {
            const int rc = record_cuda(attr);
            (void)cudaGetLastError();
            return rc;
        }
        opted_in[dev] = true;
    }
    int grid = grid_for(a.n_tiles, 1);
    if (grid < 0) return grid;
    // fewer CTAs than SMs leave the other SMs to a kernel on another stream (the pull of the next chunk)
    if (g_tune.adam_tma_ctas > 0 && g_tune.adam_tma_ctas < grid) grid = g_tune.adam_tma_ctas;
    adam_tma_kernel<DT, MATH, MM, PW, STAGES><<<grid, kTmaBlock, smem, s>>>(a);
    return record_cuda(cudaGetLastError());
}

template <int DT, int MATH, bool MM = false, int PW = 0>
int launch_adam_tma(const AdamArgs& a, cudaStream_t s) {
    constexpr int kDeepest = TmaRing<DT, MATH, PW>::kStages;
    if constexpr (kDeepest > 3) {
        if (g_tune.adam_tma_stages != 3) return launch_adam_tma_ring<DT, MATH, MM, PW, kDeepest>(a, s);
    }
    return launch_adam_tma_ring<DT, MATH, MM, PW, 3>(a, s);
}

template <int DT>
int launch_adam_dt(const AdamArgs& a, cudaStream_t s) {
    const bool precise = g_tune.math_mode == 1;
    if (a.mc_grads) {
        if constexpr (DT == ELX_F32) return ELX_ERR_DTYPE;   // the switch-side sum is used for 16-bit chunks
        else return precise ? launch_adam_tma<DT, 1, true>(a, s) : launch_adam_tma<DT, 2, true>(a, s);
    }
    if (a.pull) {
        // gradients pulled from the ranks' slabs inside the update kernel: what shared memory has room for
        if constexpr (DT == ELX_F32) return ELX_ERR_DTYPE;
        else if (a.push.world == 2) return precise ? launch_adam_tma<DT, 1, false, 2>(a, s) : launch_adam_tma<DT, 2, false, 2>(a, s);
        else return ELX_ERR_CAPACITY;
    }
    if ((g_tune.adam_variant == 1 && !a.force_direct) || a.push.world > 0 || a.shadow)
        return precise ? launch_adam_tma<DT, 1>(a, s) : launch_adam_tma<DT, 2>(a, s);
    if (g_tune.adam_threads == 256)
        return precise ? launch_adam_minb<DT, 16, 1>(a, s) : launch_adam_minb<DT, 16, 2>(a, s);
    return precise ? launch_adam_minb<DT, 8, 1>(a, s) : launch_adam_minb<DT, 8, 2>(a, s);
}

int launch_adam(const AdamArgs& a, int dtype, cudaStream_t s) {
    switch (dtype) {
        case ELX_F16: return launch_adam_dt<ELX_F16>(a, s);
        case ELX_BF16: return launch_adam_dt<ELX_BF16>(a, s);
        case ELX_F32: return launch_adam_dt<ELX_F32>(a, s);
    }
    return ELX_ERR_DTYPE;
}

}  // namespace

extern "C" {

static int adam_multi_common(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                             const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl, void* stream,
                             int force_direct, const ElxChunkDesc* shadow = nullptr) {
    if (!descs || !ctl) return ELX_ERR_NULL;
    if (shadow && !aligned(shadow, 8)) return ELX_ERR_ALIGN;
    if (n_groups > 0 && (!segs || !hyper)) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (first < 0 || count < 0 || n_tiles < 0 || n_groups < 0) return ELX_ERR_SIZE;
    if (n_groups > kMaxGroups) return ELX_ERR_CAPACITY;
    if (!aligned(descs, 8) || !aligned(ctl, 16) || (segs && !aligned(segs, 8)) || (hyper && !aligned(hyper, 4)))
        return ELX_ERR_ALIGN;
    if (count == 0 || n_tiles == 0) return ELX_OK;
    AdamArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = descs;
    a.segs = segs;
    a.hyper = hyper;
    a.ctl = ctl;
    a.first = first;
    a.count = count;
    a.n_groups = n_groups;
    a.n_tiles = n_tiles;
    a.force_direct = force_direct;
    a.shadow = shadow;
    return launch_adam(a, dtype, static_cast<cudaStream_t>(stream));
}

int elx_adam_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype, const ElxSeg* segs,
                   const ElxHyper* hyper, int n_groups, ElxCtl* ctl, void* stream) {
    return adam_multi_common(descs, first, count, n_tiles, dtype, segs, hyper, n_groups, ctl, stream, 0);
}

int elx_adam_multi_hostmem(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                           const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl, void* stream) {
    return adam_multi_common(descs, first, count, n_tiles, dtype, segs, hyper, n_groups, ctl, stream, 1);
}

int elx_adam_multi_shadow(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                          int64_t n_tiles, int dtype, const ElxSeg* segs, const ElxHyper* hyper, int n_groups,
                          ElxCtl* ctl, void* stream) {
    if (!shadow) return ELX_ERR_NULL;
    return adam_multi_common(descs, first, count, n_tiles, dtype, segs, hyper, n_groups, ctl, stream, 0, shadow);
}

static int single_pass_common(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                              int64_t n_tiles, int dtype, const ElxSeg* segs, const ElxHyper* hyper, int n_groups,
                              ElxCtl* ctl, uint32_t* chunk_flags, const ElxPeerTable* grads, const ElxPeerTable* gather,
                              const int64_t* block_off, const void* grads_mc, void* gather_mc, int repair, void* stream) {
    if (!descs || !shadow || !ctl) return ELX_ERR_NULL;
    if (!repair && n_groups > 0 && (!segs || !hyper)) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (first < 0 || count < 0 || n_tiles < 0 || n_groups < 0) return ELX_ERR_SIZE;
    if (n_groups > kMaxGroups) return ELX_ERR_CAPACITY;
    if (!aligned(descs, 8) || !aligned(shadow, 8) || !aligned(ctl, 16) || (segs && !aligned(segs, 8)) ||
        (hyper && !aligned(hyper, 4)) || (chunk_flags && !aligned(chunk_flags, 4)))
        return ELX_ERR_ALIGN;
    const bool sharded = gather && gather->world > 0;
    if (sharded) {
        if (!block_off) return ELX_ERR_NULL;
        if (!aligned(block_off, 8)) return ELX_ERR_ALIGN;
        int rc = peer_table_ok(*gather);
        if (rc != ELX_OK) return rc;
        if (!repair && (grads_mc || gather_mc)) {
            // the gradient of a shard is the sum over the ranks' slabs: both views of the slabs are needed
            if (!grads || !grads_mc || !gather_mc) return ELX_ERR_NULL;
            rc = peer_table_ok(*grads);
            if (rc != ELX_OK) return rc;
            if (grads->world != gather->world || grads->rank != gather->rank) return ELX_ERR_ARG;
            if (!aligned(grads_mc, 32) || !aligned(gather_mc, 32)) return ELX_ERR_ALIGN;
            if (dtype == ELX_F32) return ELX_ERR_DTYPE;
        }
    } else if (grads_mc || gather_mc) {
        return ELX_ERR_ARG;
    }
    if (count == 0 || n_tiles == 0) return ELX_OK;
    AdamArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = descs;
    a.shadow = shadow;
    a.segs = segs;
    a.hyper = hyper;
    a.ctl = ctl;
    a.first = first;
    a.count = count;
    a.n_groups = n_groups;
    a.n_tiles = n_tiles;
    a.spec = 1;
    a.repair = repair;
    a.chunk_flags = chunk_flags;
    if (sharded) {
        a.push = *gather;
        a.push_off = block_off;
        if (!repair && grads_mc) {
            a.grads = *grads;
            a.mc_grads = static_cast<const char*>(grads_mc);
            a.mc_gather = static_cast<char*>(gather_mc);
        }
    }
    return launch_adam(a, dtype, static_cast<cudaStream_t>(stream));
}

int elx_adam_multi_single_pass(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count,
                               int64_t n_tiles, int dtype, const ElxSeg* segs, const ElxHyper* hyper, int n_groups,
                               ElxCtl* ctl, uint32_t* chunk_flags, ElxPeerTable grads, ElxPeerTable gather,
                               const int64_t* block_off, const void* grads_mc, void* gather_mc, void* stream) {
    return single_pass_common(descs, shadow, first, count, n_tiles, dtype, segs, hyper, n_groups, ctl, chunk_flags,
                              &grads, &gather, block_off, grads_mc, gather_mc, 0, stream);
}

int elx_adam_multi_repair(const ElxChunkDesc* descs, const ElxChunkDesc* shadow, int first, int count, int64_t n_tiles,
                          int dtype, ElxCtl* ctl, ElxPeerTable gather, const int64_t* block_off, void* gather_mc,
                          void* stream) {
    (void)gather_mc;   // the rebuilt working copies go out with plain peer stores
    return single_pass_common(descs, shadow, first, count, n_tiles, dtype, nullptr, nullptr, 0, ctl, nullptr, nullptr,
                              &gather, block_off, nullptr, nullptr, 1, stream);
}

int elx_adam_multi_push(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                        const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl, ElxPeerTable gather,
                        const int64_t* block_off, void* stream) {
    if (!descs || !ctl || !block_off) return ELX_ERR_NULL;
    if (n_groups > 0 && (!segs || !hyper)) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (first < 0 || count < 0 || n_tiles < 0 || n_groups < 0) return ELX_ERR_SIZE;
    if (n_groups > kMaxGroups) return ELX_ERR_CAPACITY;
    const int rc = peer_table_ok(gather);
    if (rc != ELX_OK) return rc;
    if (!aligned(descs, 8) || !aligned(ctl, 16) || !aligned(block_off, 8) || (segs && !aligned(segs, 8)) ||
        (hyper && !aligned(hyper, 4)))
        return ELX_ERR_ALIGN;
    if (count == 0 || n_tiles == 0) return ELX_OK;
    AdamArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = descs;
    a.segs = segs;
    a.hyper = hyper;
    a.ctl = ctl;
    a.first = first;
    a.count = count;
    a.n_groups = n_groups;
    a.n_tiles = n_tiles;
    a.push = gather;
    a.push_off = block_off;
    return launch_adam(a, dtype, static_cast<cudaStream_t>(stream));
}

int elx_adam_multi_pull_push(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                             const ElxSeg* segs, const ElxHyper* hyper, int n_groups, ElxCtl* ctl, ElxPeerTable grads,
                             ElxPeerTable gather, const int64_t* block_off, void* stream) {
    if (!descs || !ctl || !block_off) return ELX_ERR_NULL;
    if (n_groups > 0 && (!segs || !hyper)) return ELX_ERR_NULL;
    if (dtype != ELX_F16 && dtype != ELX_BF16) return ELX_ERR_DTYPE;
    if (first < 0 || count < 0 || n_tiles < 0 || n_groups < 0) return ELX_ERR_SIZE;
    if (n_groups > kMaxGroups) return ELX_ERR_CAPACITY;
    int rc = peer_table_ok(gather);
    if (rc != ELX_OK) return rc;
    rc = peer_table_ok(grads);
    if (rc != ELX_OK) return rc;
    if (grads.world != gather.world || grads.rank != gather.rank) return ELX_ERR_ARG;
    if (gather.world != 2) return ELX_ERR_CAPACITY;
    if (!aligned(descs, 8) || !aligned(ctl, 16) || !aligned(block_off, 8) || (segs && !aligned(segs, 8)) ||
        (hyper && !aligned(hyper, 4)))
        return ELX_ERR_ALIGN;
    if (count == 0 || n_tiles == 0) return ELX_OK;
    AdamArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = descs;
    a.segs = segs;
    a.hyper = hyper;
    a.ctl = ctl;
    a.first = first;
    a.count = count;
    a.n_groups = n_groups;
    a.n_tiles = n_tiles;
    a.push = gather;
    a.push_off = block_off;
    a.grads = grads;
    a.pull = 1;
    return launch_adam(a, dtype, static_cast<cudaStream_t>(stream));
}

int elx_adam_chunk(float* master, float* exp_avg, float* exp_avg_sq, void* grad_param, int dtype, int64_t n_valid,
                   int64_t n_shard, ElxHyper hyper, ElxCtl* ctl, void* stream) {
    if (!master || !exp_avg || !exp_avg_sq || !grad_param || !ctl) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (n_shard < 0 || n_valid < 0 || n_valid > n_shard) return ELX_ERR_SIZE;
    if (!aligned(master, 4) || !aligned(exp_avg, 4) || !aligned(exp_avg_sq, 4) ||
        !aligned(grad_param, dtype_bytes(dtype)) || !aligned(ctl, 16))
        return ELX_ERR_ALIGN;
    if (n_shard == 0) return ELX_OK;
    AdamArgs a;
    memset(&a, 0, sizeof(a));
    a.ctl = ctl;
    a.first = 0;
    a.count = 1;
    a.n_groups = 1;
    a.inline_tables = 1;
    a.n_tiles = (n_shard + kTile - 1) / kTile;
    a.one_desc.master = master;
    a.one_desc.exp_avg = exp_avg;
    a.one_desc.exp_avg_sq = exp_avg_sq;
    a.one_desc.grad_param = grad_param;
    a.one_desc.n_shard = n_shard;
    a.one_desc.n_valid = n_valid;
    a.one_desc.tile_begin = 0;
    a.one_desc.seg_first = 0;
    a.one_desc.seg_count = n_valid > 0 ? 1 : 0;
    a.one_desc.dtype = dtype;
    a.one_seg.begin = 0;
    a.one_seg.end = n_valid;
    a.one_seg.group = 0;
    a.one_hyper = hyper;
    return launch_adam(a, dtype, static_cast<cudaStream_t>(stream));
}

int elx_cast_copyback(const float* master, void* dst, int dtype, int64_t n, void* stream) {
    if (!master || !dst) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (n < 0) return ELX_ERR_SIZE;
    if (!aligned(master, 4) || !aligned(dst, dtype_bytes(dtype))) return ELX_ERR_ALIGN;
    if (n == 0) return ELX_OK;
    const int vec_ok = aligned(master, 32) && aligned(dst, 32);
    const int grid = grid_for((n + kTile - 1) / kTile, 8);
    if (grid < 0) return grid;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case ELX_F16: cast_kernel<ELX_F16><<<grid, 256, 0, s>>>(master, dst, n, vec_ok); break;
        case ELX_BF16: cast_kernel<ELX_BF16><<<grid, 256, 0, s>>>(master, dst, n, vec_ok); break;
        case ELX_F32: cast_kernel<ELX_F32><<<grid, 256, 0, s>>>(master, dst, n, vec_ok); break;
    }
    return record_cuda(cudaGetLastError());
}

}  // extern "C"
