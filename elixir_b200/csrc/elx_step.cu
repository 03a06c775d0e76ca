// Chunk-level mixed-precision optimizer step for B200 (sm_100a): kernels and their C ABI.
//
// Everything here is HBM-bandwidth work: each element of a chunk shard is read once and written
// once, with 256-bit global accesses, from a persistent grid sized to the SM count.  There is no
// shared-memory staging and no tensor-core use: the arithmetic intensity is ~0.4 flop/byte.
//
// Kernels
//   probe_kernel     inf/nan probe of the reduced low-precision gradients (optionally fused with the
//                    copy into the shard, optionally with a fixed-order sum of squares)
//   norm_finalize    fixed-order reduction of the per-tile partial sums of squares
//   step_begin       one thread: skip decision, combined divisor, loss-scaler update, step count
//   adam_kernel      unscale + Adam/AdamW on fp32 master / exp_avg / exp_avg_sq + rounded
//                    low-precision copy-back, or copy-back only on a skipped step
//   cast_kernel      fp32 -> low-precision copy-back alone
//
// Semantics follow hpcaitech/Elixir's ElixirOptimizer.step (elixir/wrapper/optimizer.py:192-220),
// Chunk.update_extra_reduce_info / optim_update (elixir/chunk/core/chunk.py:345-356, 403-415) and
// the multi-tensor Adam (with div_scale) and DynamicGradScaler of ColossalAI that Elixir calls.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "elixir_b200.h"

namespace {

constexpr int kTile = ELX_TILE;
constexpr int kMaxGroups = 64;
constexpr int kProbeThreads = 256;   // 16 elements per thread and tile

// ------------------------------------------------------------------------------------------------
// host-side state
// ------------------------------------------------------------------------------------------------

thread_local char t_cuda_err[256] = "";

// Launch-shape knobs (elx_set_tuning).  A CTAs-per-SM cap of 0 means "as many as are resident".
struct Tuning {
    int adam_threads = 256;
    int adam_min_blocks = 2;      // __launch_bounds__ minimum CTAs per SM the kernel is compiled for
    int adam_ctas_per_sm = 0;
    int probe_ctas_per_sm = 0;
    int probe_unroll = 4;
    int math_mode = 1;
    int adam_variant = 1;         // 0 = direct global accesses, 1 = bulk-copy (TMA) pipeline
    int pull_ctas_per_sm = 0;
};
Tuning g_tune;

// CTAs of `kernel` that fit on one SM (cached per kernel instantiation by the callers).
template <typename KernelT>
int resident_ctas(KernelT kernel, int threads) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        n = 1;
    }
    return n;
}

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

inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline bool dtype_ok(int dt) { return dt == ELX_F16 || dt == ELX_BF16 || dt == ELX_F32; }
inline int dtype_bytes(int dt) { return dt == ELX_F32 ? 4 : 2; }

// ------------------------------------------------------------------------------------------------
// 256-bit / 128-bit global accesses with streaming hints (data is touched once per step)
// ------------------------------------------------------------------------------------------------

struct U8 {
    uint32_t x[8];
};

__device__ __forceinline__ U8 ld256(const void* p) {
    U8 r;
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.x[0]), "=r"(r.x[1]), "=r"(r.x[2]), "=r"(r.x[3]), "=r"(r.x[4]), "=r"(r.x[5]),
                   "=r"(r.x[6]), "=r"(r.x[7])
                 : "l"(p));
    return r;
}

__device__ __forceinline__ void st256(void* p, const U8& v) {
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :
                 : "l"(p), "r"(v.x[0]), "r"(v.x[1]), "r"(v.x[2]), "r"(v.x[3]), "r"(v.x[4]), "r"(v.x[5]),
                   "r"(v.x[6]), "r"(v.x[7])
                 : "memory");
}

struct U4 {
    uint32_t x[4];
};

__device__ __forceinline__ U4 ld128(const void* p) {
    U4 r;
    asm volatile("ld.global.cs.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x[0]), "=r"(r.x[1]), "=r"(r.x[2]), "=r"(r.x[3])
                 : "l"(p));
    return r;
}

__device__ __forceinline__ void st128(void* p, const U4& v) {
    asm volatile("st.global.cs.v4.b32 [%0], {%1,%2,%3,%4};"
                 :
                 : "l"(p), "r"(v.x[0]), "r"(v.x[1]), "r"(v.x[2]), "r"(v.x[3])
                 : "memory");
}

// N consecutive 32-bit words, N in {4, 8, 16}
template <int N>
__device__ __forceinline__ void ld_words(const void* p, uint32_t (&w)[N]) {
    if constexpr (N == 4) {
        U4 r = ld128(p);
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = r.x[i];
    } else {
#pragma unroll
        for (int k = 0; k < N / 8; ++k) {
            U8 r = ld256(static_cast<const char*>(p) + 32 * k);
#pragma unroll
            for (int i = 0; i < 8; ++i) w[8 * k + i] = r.x[i];
        }
    }
}

template <int N>
__device__ __forceinline__ void st_words(void* p, const uint32_t (&w)[N]) {
    if constexpr (N == 4) {
        U4 r;
#pragma unroll
        for (int i = 0; i < 4; ++i) r.x[i] = w[i];
        st128(p, r);
    } else {
#pragma unroll
        for (int k = 0; k < N / 8; ++k) {
            U8 r;
#pragma unroll
            for (int i = 0; i < 8; ++i) r.x[i] = w[8 * k + i];
            st256(static_cast<char*>(p) + 32 * k, r);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// low-precision element traits
// ------------------------------------------------------------------------------------------------

template <int DT>
struct Lp;

template <>
struct Lp<ELX_F16> {
    using T = __half;
    static constexpr int kBytes = 2;
    static __device__ __forceinline__ float2 unpack2(uint32_t u) {
        return __half22float2(*reinterpret_cast<const __half2*>(&u));
    }
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    // non-zero iff one of the two packed values has an all-ones exponent (inf or nan)
    static __device__ __forceinline__ uint32_t nonfinite_word(uint32_t u) {
        return ((u & 0x7C007C00u) + 0x04000400u) & 0x80008000u;
    }
    static __device__ __forceinline__ bool nonfinite(T v) { return (__half_as_ushort(v) & 0x7C00u) == 0x7C00u; }
    static __device__ __forceinline__ float to_float(T v) { return __half2float(v); }
    static __device__ __forceinline__ T from_float(float f) { return __float2half_rn(f); }
};

template <>
struct Lp<ELX_BF16> {
    using T = __nv_bfloat16;
    static constexpr int kBytes = 2;
    static __device__ __forceinline__ float2 unpack2(uint32_t u) {
        // bf16 -> fp32 is a 16-bit shift
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
    }
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ uint32_t nonfinite_word(uint32_t u) {
        return ((u & 0x7F807F80u) + 0x00800080u) & 0x80008000u;
    }
    static __device__ __forceinline__ bool nonfinite(T v) { return (__bfloat16_as_ushort(v) & 0x7F80u) == 0x7F80u; }
    static __device__ __forceinline__ float to_float(T v) { return __bfloat162float(v); }
    static __device__ __forceinline__ T from_float(float f) { return __float2bfloat16_rn(f); }
};

template <>
struct Lp<ELX_F32> {
    using T = float;
    static constexpr int kBytes = 4;
    static __device__ __forceinline__ uint32_t nonfinite_word(uint32_t u) {
        return (u & 0x7F800000u) == 0x7F800000u ? 1u : 0u;
    }
    static __device__ __forceinline__ bool nonfinite(T v) {
        return (__float_as_uint(v) & 0x7F800000u) == 0x7F800000u;
    }
    static __device__ __forceinline__ float to_float(T v) { return v; }
    static __device__ __forceinline__ T from_float(float f) { return f; }
};

// Work split inside a tile.  A thread owns EPT/8 groups of 8 consecutive elements.  A warp owns a
// slab of 32 * EPT consecutive elements; group j of lane l starts at j * 256 + l * 8 inside the slab,
// so every warp-wide access (256-bit per lane on the fp32 arrays, 128-bit per lane on the 16-bit
// array) covers whole, consecutive 128-byte lines.
template <int EPT>
__device__ __forceinline__ int group_offset(int j) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    return warp * (32 * EPT) + j * 256 + lane * 8;
}

// The thread's EPT low-precision elements of the tile starting at element e0, as fp32.
template <int DT, int EPT>
__device__ __forceinline__ void load_lowp(const void* base, int64_t e0, float (&g)[EPT]) {
#pragma unroll
    for (int j = 0; j < EPT / 8; ++j) {
        const int64_t idx = e0 + group_offset<EPT>(j);
        if constexpr (DT == ELX_F32) {
            const U8 r = ld256(static_cast<const float*>(base) + idx);
#pragma unroll
            for (int i = 0; i < 8; ++i) g[8 * j + i] = __uint_as_float(r.x[i]);
        } else {
            const U4 r = ld128(static_cast<const uint16_t*>(base) + idx);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = Lp<DT>::unpack2(r.x[i]);
                g[8 * j + 2 * i] = f.x;
                g[8 * j + 2 * i + 1] = f.y;
            }
        }
    }
}

template <int DT, int EPT>
__device__ __forceinline__ void store_lowp(void* base, int64_t e0, const float (&p)[EPT]) {
#pragma unroll
    for (int j = 0; j < EPT / 8; ++j) {
        const int64_t idx = e0 + group_offset<EPT>(j);
        if constexpr (DT == ELX_F32) {
            U8 r;
#pragma unroll
            for (int i = 0; i < 8; ++i) r.x[i] = __float_as_uint(p[8 * j + i]);
            st256(static_cast<float*>(base) + idx, r);
        } else {
            U4 r;
#pragma unroll
            for (int i = 0; i < 4; ++i) r.x[i] = Lp<DT>::pack2(p[8 * j + 2 * i], p[8 * j + 2 * i + 1]);
            st128(static_cast<uint16_t*>(base) + idx, r);
        }
    }
}

template <int EPT>
__device__ __forceinline__ void load_f32(const float* base, int64_t e0, float (&v)[EPT]) {
#pragma unroll
    for (int j = 0; j < EPT / 8; ++j) {
        const U8 r = ld256(base + e0 + group_offset<EPT>(j));
#pragma unroll
        for (int i = 0; i < 8; ++i) v[8 * j + i] = __uint_as_float(r.x[i]);
    }
}

template <int EPT>
__device__ __forceinline__ void store_f32(float* base, int64_t e0, const float (&v)[EPT]) {
#pragma unroll
    for (int j = 0; j < EPT / 8; ++j) {
        U8 r;
#pragma unroll
        for (int i = 0; i < 8; ++i) r.x[i] = __float_as_uint(v[8 * j + i]);
        st256(base + e0 + group_offset<EPT>(j), r);
    }
}

// ------------------------------------------------------------------------------------------------
// tile -> chunk and element -> segment lookup, cached across a CTA's consecutive tiles
// ------------------------------------------------------------------------------------------------

// The descriptor a CTA is working in lives in shared memory: every thread of a CTA handles the same
// tile, so one thread searches and the others read the result.  The search reruns only when a tile
// leaves the cached descriptor (once per chunk for most CTAs).
struct ChunkCursor {
    int64_t t0, t1;   // tile range of the cached descriptor
    int index;
    int vec_ok;       // all four pointers are 32-byte aligned
    ElxChunkDesc d;
};

__device__ __forceinline__ int64_t tiles_of(int64_t n) { return (n + kTile - 1) / kTile; }

__device__ __forceinline__ void cursor_reset(ChunkCursor& cur) {
    if (threadIdx.x == 0) {
        cur.t0 = cur.t1 = 0;
        cur.index = -1;
        cur.vec_ok = 0;
    }
    __syncthreads();
}

// CTA-collective (every thread calls it with the same t).  cur is in shared memory.
__device__ __forceinline__ bool locate_chunk(const ElxChunkDesc* __restrict__ descs, int first, int count,
                                             int64_t t, ChunkCursor& cur) {
    if (t >= cur.t0 && t < cur.t1) return true;
    __syncthreads();   // nobody still reads the old cursor
    if (threadIdx.x == 0) {
        int lo = first, hi = first + count - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (descs[mid].tile_begin <= t) lo = mid; else hi = mid - 1;
        }
        const ElxChunkDesc d = descs[lo];
        const int64_t t0 = d.tile_begin, t1 = t0 + tiles_of(d.n_shard);
        if (t >= t0 && t < t1) {
            cur.d = d;
            cur.index = lo;
            cur.t0 = t0;
            cur.t1 = t1;
            const uintptr_t bits = reinterpret_cast<uintptr_t>(d.master) | reinterpret_cast<uintptr_t>(d.exp_avg) |
                                   reinterpret_cast<uintptr_t>(d.exp_avg_sq) |
                                   reinterpret_cast<uintptr_t>(d.grad_param);
            cur.vec_ok = (bits & 31u) == 0;
        }
    }
    __syncthreads();
    return t >= cur.t0 && t < cur.t1;
}

// Cached segment of the cached chunk, also in shared memory.
struct SegCursor {
    int64_t b, e;   // [b, e) of the cached segment, b == e when none
    int group;
    int chunk;      // descriptor index the cache belongs to
};

// Index (relative to the chunk's first segment) of the last segment with begin <= e, or -1.
__device__ __forceinline__ int find_seg(const ElxSeg* __restrict__ segs, int n, int64_t e) {
    int lo = 0, hi = n;   // first segment with begin > e
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (segs[mid].begin <= e) lo = mid + 1; else hi = mid;
    }
    return lo - 1;
}

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

// How the gradient is unscaled in this launch.
enum { kNoDiv = 0, kMulInv = 1, kTrueDiv = 2 };

template <int MATH>
__device__ __forceinline__ void adam_elem(float& p, float& m, float& v, float g, const GroupK& k, int div_mode,
                                          float div, float inv_div) {
    if (div_mode == kMulInv) g *= inv_div;                    // exact: the divisor is a power of two
    else if (div_mode == kTrueDiv) g = __fdiv_rn(g, div);
    g = fmaf(k.wd_l2, p, g);
    m = fmaf(k.beta1, m, k.omb1 * g);
    v = fmaf(k.beta2, v, (k.omb2 * g) * g);
    float upd;
    if constexpr (MATH == 1) {
        float mhat = __fdiv_rn(m, k.bc1);
        float vhat = __fdiv_rn(v, k.bc2);
        float denom = __fsqrt_rn(vhat) + k.eps;
        upd = __fdiv_rn(mhat, denom);
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
                                               ChunkCursor& s_cur) {
    bool bad_desc = false;
    const int64_t tile_lo = descs[a.first].tile_begin;
    for (int64_t it = blockIdx.x; it < a.n_tiles; it += gridDim.x) {
        const int64_t t = tile_lo + it;
        if (!locate_chunk(descs, a.first, a.count, t, s_cur) || s_cur.d.dtype != DT) {
            bad_desc = true;
            continue;
        }
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
            for (int64_t e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
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
        bad_desc = copyback_tiles<DT, EPT>(a, descs, s_cur);
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
            load_lowp<DT, EPT>(lowp, e0, g);
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
        } else {
            // ragged tile: shard tail, segment boundary, uncovered elements or unaligned pointers
            typename Lp<DT>::T* gp = static_cast<typename Lp<DT>::T*>(lowp);
            for (int64_t e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
                float p = master[e];
                const int si = find_seg(csegs, n_segs, e);
                if (si >= 0 && e < csegs[si].end) {
                    const int ge = csegs[si].group;
                    if (ge >= 0 && ge < a.n_groups) {
                        const GroupK k = s_group[ge];
                        float g = Lp<DT>::to_float(gp[e]);
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
// Same arithmetic, different data movement: one elected thread streams whole tiles between HBM and
// shared memory with cp.async.bulk (the TMA unit's untiled form), completion tracked by mbarriers,
// so loads of the next two tiles and stores of the previous one are in flight while the CTA's warps
// compute on the current one out of shared memory.  One CTA per SM, kTmaStages stages of one tile
// each (16-bit gradients: 8 KB + 3 x 16 KB = 56 KB per stage).
//
//   iteration k (stage s = k % 3):
//     all threads   wait full[s]; read g,p,m,v from the stage; update; write p,m,v,p16 back in place
//                   fence.proxy.async; __syncthreads
//     thread 0      4 bulk stores stage s -> HBM, commit; wait until the stores of iteration k-1 have
//                   read their stage; arm full[(k+2) % 3] and issue the 4 bulk loads of tile k+2 into it
//
// Ragged tiles (shard tail, segment boundary, unaligned pointers) bypass the pipeline and are updated
// in place in global memory by the same scalar path as the direct kernel.  Every mbarrier wait is
// bounded: on expiry the CTA raises ELX_STAT_TIMEOUT, stops issuing copies, drains and returns.

constexpr int kTmaStages = 3;
constexpr int kTmaThreads = 512;
constexpr uint32_t kTmaSpinLimit = 1u << 22;   // polls of at most ~1 us each: a few seconds, then give up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)   // give up this poll after about a microsecond
        : "memory");
    return done != 0;
}
// false = gave up
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kTmaSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

enum { kTileNone = 0, kTileBulk = 1, kTileRagged = 2, kTileBad = 3 };

// What the producer thread decided about one tile, published to the CTA through shared memory.
struct TileSlot {
    float* master;
    float* exp_avg;
    float* exp_avg_sq;
    void* lowp;
    const ElxSeg* segs;
    int64_t e0, e1;
    int64_t push_elem;   // element offset of this tile inside every rank's gather slab (push all-gather)
    int n_segs;
    int group;
    int kind;
    int pad;
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
    int64_t seg_b = 0, seg_e = 0;
    int seg_group = -1;
    int seg_chunk = -1;
};

template <int DT>
__device__ __forceinline__ void classify_tile(const AdamArgs& a, const ElxChunkDesc* __restrict__ descs,
                                              const ElxSeg* __restrict__ segs, int64_t t, ProducerCursor& pc,
                                              TileSlot& out) {
    if (!(t >= pc.t0 && t < pc.t1)) {
        int lo = a.first, hi = a.first + a.count - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (descs[mid].tile_begin <= t) lo = mid; else hi = mid - 1;
        }
        pc.d = descs[lo];
        pc.index = lo;
        pc.t0 = pc.d.tile_begin;
        pc.t1 = pc.t0 + tiles_of(pc.d.n_shard);
        const uintptr_t bits = reinterpret_cast<uintptr_t>(pc.d.master) | reinterpret_cast<uintptr_t>(pc.d.exp_avg) |
                               reinterpret_cast<uintptr_t>(pc.d.exp_avg_sq) |
                               reinterpret_cast<uintptr_t>(pc.d.grad_param);
        pc.vec_ok = (bits & 31u) == 0;
    }
    if (!(t >= pc.t0 && t < pc.t1) || pc.d.dtype != DT) {
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
    out.lowp = pc.d.grad_param;
    out.segs = csegs;
    out.n_segs = pc.d.seg_count;
    out.e0 = e0;
    out.e1 = e1;
    out.group = pc.seg_group;
    out.push_elem = a.push.world > 0 ? push_base_elem(a, pc.index, pc.d.n_shard) + e0 : 0;
    const bool push_ok = a.push.world == 0 || (out.push_elem & 15) == 0;   // bulk copies need 16-byte alignment
    out.kind = (e1 - e0 == kTile && pc.vec_ok && one_group && push_ok) ? kTileBulk : kTileRagged;
}

template <int DT, int MATH>
__global__ void __launch_bounds__(kTmaThreads, 1) adam_tma_kernel(const __grid_constant__ AdamArgs a) {
    using Stage = TmaStage<DT>;
    extern __shared__ __align__(128) unsigned char s_dyn[];
    __shared__ GroupK s_group[kMaxGroups];
    __shared__ TileSlot s_slot[kTmaStages];
    __shared__ __align__(8) uint64_t s_full[kTmaStages];
    __shared__ int s_abort;

    const ElxChunkDesc* __restrict__ descs = a.inline_tables ? &a.one_desc : a.descs;
    const ElxSeg* __restrict__ segs = a.inline_tables ? &a.one_seg : a.segs;
    const ElxHyper* __restrict__ hyper = a.inline_tables ? &a.one_hyper : a.hyper;
    ElxCtl* ctl = a.ctl;

    if (ctl->skip != 0) {
        // skipped step: copy-back only, with direct accesses (6 bytes per element, no staging needed)
        __shared__ ChunkCursor s_cur;
        cursor_reset(s_cur);
        const bool bad = copyback_tiles<DT, kTile / kTmaThreads>(a, descs, s_cur);
        if (__ballot_sync(0xFFFFFFFFu, bad) && (threadIdx.x & 31) == 0) atomicOr(&ctl->status, ELX_STAT_BAD_DESC);
        return;
    }

    const float div = ctl->div_scale;
    const float inv_div = ctl->inv_div;
    const int div_mode = div > 0.0f ? (inv_div != 0.0f ? kMulInv : kTrueDiv) : kNoDiv;
    const int step = ctl->step;
    for (int gi = threadIdx.x; gi < a.n_groups; gi += blockDim.x) s_group[gi] = derive_group(hyper[gi], step);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTmaStages; ++s) mbar_init(&s_full[s], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t tile_lo = descs[a.first].tile_begin;
    const int64_t my_tiles = blockIdx.x < a.n_tiles ? (a.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    ProducerCursor pc;
    float nan_acc = 0.0f;
    bool bad_desc = false;

    // producer: classify tile k of this CTA, publish it in its stage's slot, start its loads
    auto produce = [&](int64_t k) {
        const int s = static_cast<int>(k % kTmaStages);
        TileSlot slot;
        slot.kind = kTileNone;
        classify_tile<DT>(a, descs, segs, tile_lo + blockIdx.x + k * gridDim.x, pc, slot);
        s_slot[s] = slot;
        if (slot.kind == kTileBulk) {
            unsigned char* base = s_dyn + static_cast<size_t>(s) * Stage::kBytes;
            mbar_arrive_expect_tx(&s_full[s], Stage::kBytes);
            bulk_g2s(base, static_cast<const char*>(slot.lowp) + slot.e0 * Lp<DT>::kBytes, Stage::kLowpBytes, &s_full[s]);
            bulk_g2s(base + Stage::kLowpBytes, slot.master + slot.e0, Stage::kF32Bytes, &s_full[s]);
            bulk_g2s(base + Stage::kLowpBytes + Stage::kF32Bytes, slot.exp_avg + slot.e0, Stage::kF32Bytes, &s_full[s]);
            bulk_g2s(base + Stage::kLowpBytes + 2 * Stage::kF32Bytes, slot.exp_avg_sq + slot.e0, Stage::kF32Bytes,
                     &s_full[s]);
        } else {
            mbar_arrive(&s_full[s]);   // nothing to load: the phase completes at once and publishes the slot
        }
    };

    if (threadIdx.x == 0) {
        for (int64_t k = 0; k < my_tiles && k < kTmaStages - 1; ++k) produce(k);
    }

    int64_t k = 0;
    for (; k < my_tiles; ++k) {
        const int s = static_cast<int>(k % kTmaStages);
        const uint32_t parity = static_cast<uint32_t>((k / kTmaStages) & 1);
        if (!mbar_wait_bounded(&s_full[s], parity)) s_abort = 1;
        __syncthreads();
        if (s_abort) break;
        const TileSlot slot = s_slot[s];
        unsigned char* base = s_dyn + static_cast<size_t>(s) * Stage::kBytes;

        if (slot.kind == kTileBulk) {
            const GroupK k_ = s_group[slot.group];
            float* sp = reinterpret_cast<float*>(base + Stage::kLowpBytes);
            float* sm = sp + kTile;
            float* sv = sm + kTile;
            // a thread owns 2 x 4 consecutive elements, 2048 apart: conflict-free 128-bit shared accesses
#pragma unroll
            for (int h = 0; h < kTile / (kTmaThreads * 4); ++h) {
                const int e = h * (kTmaThreads * 4) + threadIdx.x * 4;
                float4 p = *reinterpret_cast<float4*>(sp + e);
                float4 m = *reinterpret_cast<float4*>(sm + e);
                float4 v = *reinterpret_cast<float4*>(sv + e);
                float g[4];
                if constexpr (DT == ELX_F32) {
                    const float4 gg = *reinterpret_cast<const float4*>(base + static_cast<size_t>(e) * 4);
                    g[0] = gg.x; g[1] = gg.y; g[2] = gg.z; g[3] = gg.w;
                } else {
                    const uint2 gg = *reinterpret_cast<const uint2*>(base + static_cast<size_t>(e) * 2);
                    const float2 a0 = Lp<DT>::unpack2(gg.x), a1 = Lp<DT>::unpack2(gg.y);
                    g[0] = a0.x; g[1] = a0.y; g[2] = a1.x; g[3] = a1.y;
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
                }
            }
            fence_async_smem();   // the bulk stores below read what the threads just wrote
        } else if (slot.kind == kTileRagged) {
            typename Lp<DT>::T* gp = static_cast<typename Lp<DT>::T*>(slot.lowp);
            for (int64_t e = slot.e0 + threadIdx.x; e < slot.e1; e += blockDim.x) {
                float p = slot.master[e];
                const int si = find_seg(slot.segs, slot.n_segs, e);
                if (si >= 0 && e < slot.segs[si].end) {
                    const int ge = slot.segs[si].group;
                    if (ge >= 0 && ge < a.n_groups) {
                        const GroupK k_ = s_group[ge];
                        float g = Lp<DT>::to_float(gp[e]);
                        float m = slot.exp_avg[e], v = slot.exp_avg_sq[e];
                        nan_acc = fmaf(0.0f, g, nan_acc);
                        adam_elem<MATH>(p, m, v, g, k_, div_mode, div, inv_div);
                        slot.master[e] = p;
                        slot.exp_avg[e] = m;
                        slot.exp_avg_sq[e] = v;
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
        __syncthreads();   // the stage is fully written (bulk) / fully consumed

        if (threadIdx.x == 0) {
            if (slot.kind == kTileBulk) {
                bulk_s2g(static_cast<char*>(slot.lowp) + slot.e0 * Lp<DT>::kBytes, base, Stage::kLowpBytes);
                bulk_s2g(slot.master + slot.e0, base + Stage::kLowpBytes, Stage::kF32Bytes);
                bulk_s2g(slot.exp_avg + slot.e0, base + Stage::kLowpBytes + Stage::kF32Bytes, Stage::kF32Bytes);
                bulk_s2g(slot.exp_avg_sq + slot.e0, base + Stage::kLowpBytes + 2 * Stage::kF32Bytes, Stage::kF32Bytes);
                // push all-gather: the same 8 KB of refreshed parameters to every rank's gather block,
                // plain (non-multicast) bulk stores, W - 1 of them crossing NVLink
                for (int j = 0; j < a.push.world; ++j)
                    bulk_s2g(static_cast<char*>(a.push.base[j]) + slot.push_elem * Lp<DT>::kBytes, base,
                             Stage::kLowpBytes);
            }
            bulk_commit();
            if (k + kTmaStages - 1 < my_tiles) {
                bulk_wait_read<1>();   // the stage of tile k-1 has been read out by its stores
                produce(k + kTmaStages - 1);
            }
        }
    }
    if (threadIdx.x == 0) {
        if (s_abort) {
            // gave up on tile k: the loads already issued for the tiles after it still target this CTA's
            // shared memory, so wait (bounded again) for them before the CTA may exit
            for (int64_t j = k; j < my_tiles && j < k + kTmaStages - 1; ++j)
                (void)mbar_wait_bounded(&s_full[j % kTmaStages], static_cast<uint32_t>((j / kTmaStages) & 1));
            atomicOr(&ctl->status, ELX_STAT_TIMEOUT);
        }
        bulk_wait_all();
    }

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

// ------------------------------------------------------------------------------------------------
// probe (+ copy, + sum of squares)
// ------------------------------------------------------------------------------------------------

struct ProbeArgs {
    const ElxChunkDesc* descs;
    uint32_t* chunk_flags;   // indexed by descriptor index, may be null
    uint32_t* one_flag;      // single-shard form, may be null
    ElxCtl* ctl;             // may be null
    float* scratch;          // per-tile partial sums of squares (NORM only)
    void* copy_dst;          // COPY only (single-shard form)
    int first, count, inline_tables, pad;
    int64_t n_tiles;
    ElxChunkDesc one_desc;
};

// kProbeUnroll = tiles whose loads are in flight together in one CTA iteration
template <int DT, bool COPY, bool NORM, int kProbeUnroll>
__global__ void __launch_bounds__(kProbeThreads) probe_kernel(const __grid_constant__ ProbeArgs a) {
    constexpr int EPT = kTile / kProbeThreads;                   // 16
    constexpr int WORDS = EPT * Lp<DT>::kBytes / 4;              // 8 (16-bit) or 16 (fp32)
    using T = typename Lp<DT>::T;
    __shared__ float s_part[kProbeUnroll][kProbeThreads / 32];

    const ElxChunkDesc* __restrict__ descs = a.inline_tables ? &a.one_desc : a.descs;
    const int64_t tile_lo = descs[a.first].tile_begin;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ ChunkCursor s_cur;
    cursor_reset(s_cur);
    bool bad_desc = false;

    const int64_t n_groups_of_tiles = (a.n_tiles + kProbeUnroll - 1) / kProbeUnroll;
    for (int64_t q = blockIdx.x; q < n_groups_of_tiles; q += gridDim.x) {
        uint32_t w[kProbeUnroll][WORDS];
        bool vec[kProbeUnroll];
        bool probed[kProbeUnroll];
        int chunk_of[kProbeUnroll];
        float sq[kProbeUnroll];
        uint32_t bad[kProbeUnroll];

        // issue every load of the group first, so that they are all in flight together
#pragma unroll
        for (int j = 0; j < kProbeUnroll; ++j) {
            vec[j] = false;
            probed[j] = false;
            chunk_of[j] = -1;
            sq[j] = 0.0f;
            bad[j] = 0;
            const int64_t it = q * kProbeUnroll + j;
            if (it >= a.n_tiles) continue;
            const int64_t t = tile_lo + it;
            if (!locate_chunk(descs, a.first, a.count, t, s_cur) || s_cur.d.dtype != DT) {
                bad_desc = true;
                continue;
            }
            chunk_of[j] = s_cur.index;
            struct { const void* grad_param; int64_t n_shard, n_valid; } d = {s_cur.d.grad_param, s_cur.d.n_shard,
                                                                              s_cur.d.n_valid};
            const int64_t e0 = (t - s_cur.t0) * kTile;
            const bool dst_ok = !COPY || (reinterpret_cast<uintptr_t>(a.copy_dst) & 31u) == 0;
            const bool src_ok = (reinterpret_cast<uintptr_t>(d.grad_param) & 31u) == 0;
            const bool all_valid = e0 + kTile <= d.n_valid;     // every element is probed
            const bool none_valid = e0 >= d.n_valid;            // padding only: copied, never probed
            if (!COPY && none_valid) continue;
            if (src_ok && dst_ok && e0 + kTile <= d.n_shard && (all_valid || none_valid)) {
                vec[j] = true;
                probed[j] = all_valid;
                ld_words<WORDS>(static_cast<const char*>(d.grad_param) +
                                    (e0 + static_cast<int64_t>(threadIdx.x) * EPT) * Lp<DT>::kBytes, w[j]);
            } else {
                // ragged tile: probe [e0, n_valid), copy [e0, n_shard)
                const T* src = static_cast<const T*>(d.grad_param);
                const int64_t e1 = min(e0 + kTile, d.n_shard);
                for (int64_t e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
                    const T x = src[e];
                    if (e < d.n_valid) {
                        if (Lp<DT>::nonfinite(x)) bad[j] = 1;
                        if (NORM) {
                            const float f = Lp<DT>::to_float(x);
                            sq[j] = fmaf(f, f, sq[j]);
                        }
                    }
                    if (COPY) static_cast<T*>(a.copy_dst)[e] = x;
                }
            }
        }

#pragma unroll
        for (int j = 0; j < kProbeUnroll; ++j) {
            if (vec[j]) {
                uint32_t acc = 0;
#pragma unroll
                for (int i = 0; i < WORDS; ++i) acc |= Lp<DT>::nonfinite_word(w[j][i]);
                bad[j] = probed[j] ? acc : 0u;
                if (NORM && probed[j]) {
                    float s = 0.0f;
#pragma unroll
                    for (int i = 0; i < WORDS; ++i) {
                        if constexpr (DT == ELX_F32) {
                            const float f = __uint_as_float(w[j][i]);
                            s = fmaf(f, f, s);
                        } else {
                            const float2 f = Lp<DT>::unpack2(w[j][i]);
                            s = fmaf(f.x, f.x, s);
                            s = fmaf(f.y, f.y, s);
                        }
                    }
                    sq[j] = s;
                }
                if (COPY) {
                    const int64_t it = q * kProbeUnroll + j;
                    // single-shard form: tile index == it
                    st_words<WORDS>(static_cast<char*>(a.copy_dst) +
                                        (it * kTile + static_cast<int64_t>(threadIdx.x) * EPT) * Lp<DT>::kBytes, w[j]);
                }
            }
            // warp-reduced overflow report
            const unsigned any_bad = __ballot_sync(0xFFFFFFFFu, bad[j] != 0);
            if (any_bad && lane == 0 && chunk_of[j] >= 0) {
                if (a.chunk_flags) atomicOr(&a.chunk_flags[chunk_of[j]], 1u);
                if (a.one_flag) atomicOr(a.one_flag, 1u);
                if (a.ctl) atomicOr(&a.ctl->found_inf, 1u);
            }
        }

        if (NORM) {
            // fixed-order block reduction of each tile's partial: lanes, then warps 0..7
#pragma unroll
            for (int j = 0; j < kProbeUnroll; ++j) {
                float s = sq[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xFFFFFFFFu, s, o);
                if (lane == 0) s_part[j][warp] = s;
            }
            __syncthreads();
            if (threadIdx.x < kProbeUnroll) {
                const int64_t it = q * kProbeUnroll + threadIdx.x;
                if (it < a.n_tiles) {
                    float s = 0.0f;
                    for (int wi = 0; wi < kProbeThreads / 32; ++wi) s += s_part[threadIdx.x][wi];
                    a.scratch[it] = s;
                }
            }
            __syncthreads();
        }
    }

    const unsigned ballot_desc = __ballot_sync(0xFFFFFFFFu, bad_desc);
    if (ballot_desc && lane == 0 && a.ctl) atomicOr(&a.ctl->status, ELX_STAT_BAD_DESC);
}

struct NormArgs {
    const ElxChunkDesc* descs;
    const float* scratch;
    float* chunk_l2sq;   // indexed by descriptor index, may be null
    float* one_l2sq;     // single-shard form
    float* total_l2sq;   // may be null
    int first, count, inline_tables, pad;
    ElxChunkDesc one_desc;
};

// One CTA.  Sums each descriptor's per-tile partials in a fixed order (strided per thread, then a
// binary tree over threads) in double, so that the result does not depend on the probe grid.
__global__ void __launch_bounds__(256) norm_finalize(const __grid_constant__ NormArgs a) {
    __shared__ double s_red[256];
    const ElxChunkDesc* __restrict__ descs = a.inline_tables ? &a.one_desc : a.descs;
    const int64_t tile_lo = descs[a.first].tile_begin;
    double total = 0.0;
    for (int c = a.first; c < a.first + a.count; ++c) {
        const int64_t b = descs[c].tile_begin - tile_lo;
        const int64_t n = tiles_of(descs[c].n_shard);
        double s = 0.0;
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s += static_cast<double>(a.scratch[b + i]);
        s_red[threadIdx.x] = s;
        __syncthreads();
        for (int o = 128; o > 0; o >>= 1) {
            if (threadIdx.x < o) s_red[threadIdx.x] += s_red[threadIdx.x + o];
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            const double r = s_red[0];
            if (a.chunk_l2sq) a.chunk_l2sq[c] = static_cast<float>(r);
            if (a.one_l2sq) *a.one_l2sq = static_cast<float>(r);
            total += r;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0 && a.total_l2sq) *a.total_l2sq = static_cast<float>(total);
}

// ------------------------------------------------------------------------------------------------
// NVLink: pull reduce-scatter fused with the probe, and the cross-rank barrier
// ------------------------------------------------------------------------------------------------
//
// Every rank keeps its replicated gradient blocks in a slab that all ranks of the box can address
// (peer-mapped memory).  Rank r produces its shard of a chunk by READING the r-th slice of that
// chunk's block from every rank with ordinary loads (its own slice from local HBM, W - 1 slices over
// NVLink), summing float(x) * (1/W) in rank order in fp32, rounding once to the chunk dtype, storing
// the shard and probing the rounded result for inf/nan in the same pass.  No TMA, no multicast.

struct PullArgs {
    const ElxChunkDesc* descs;
    uint32_t* chunk_flags;
    ElxCtl* ctl;
    ElxPeerTable grads;
    const int64_t* block_off;   // per descriptor: element offset of the chunk's block inside the slabs
    int first, count;
    int64_t n_tiles;
};

// kWorld > 0: the group size is a compile-time constant, so the loads from all ranks are issued back to
// back before the first one is consumed (kWorld x 32 bytes in flight per thread); 0 = any group size.
template <int DT, int kWorld>
__global__ void __launch_bounds__(256) pull_reduce_kernel(const __grid_constant__ PullArgs a) {
    constexpr int EPT = 16;                                      // consecutive elements per thread
    constexpr int WORDS = EPT * Lp<DT>::kBytes / 4;              // 8 (16-bit) or 16 (fp32)
    using T = typename Lp<DT>::T;
    __shared__ ChunkCursor s_cur;
    cursor_reset(s_cur);
    const ElxChunkDesc* __restrict__ descs = a.descs;
    const int64_t tile_lo = descs[a.first].tile_begin;
    const int world = kWorld > 0 ? kWorld : a.grads.world;
    const int rank = a.grads.rank;
    const float inv_w = 1.0f / static_cast<float>(world);
    const int lane = threadIdx.x & 31;
    bool bad_desc = false;

    for (int64_t it = blockIdx.x; it < a.n_tiles; it += gridDim.x) {
        const int64_t t = tile_lo + it;
        if (!locate_chunk(descs, a.first, a.count, t, s_cur) || s_cur.d.dtype != DT) {
            bad_desc = true;
            continue;
        }
        const int64_t n_shard = s_cur.d.n_shard, n_valid = s_cur.d.n_valid;
        const int64_t e0 = (t - s_cur.t0) * kTile;
        const int64_t e1 = min(e0 + kTile, n_shard);
        const int64_t src0 = a.block_off[s_cur.index] + static_cast<int64_t>(rank) * n_shard;   // element offset
        void* const dst = s_cur.d.grad_param;
        const bool all_valid = e0 + kTile <= n_valid, none_valid = e0 >= n_valid;
        uint32_t bad = 0;
        if ((e1 - e0 == kTile) && (all_valid || none_valid) && (src0 & 15) == 0 &&
            (reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
            const int64_t mine = e0 + static_cast<int64_t>(threadIdx.x) * EPT;
            float acc[EPT];
#pragma unroll
            for (int i = 0; i < EPT; ++i) acc[i] = 0.0f;
            auto accumulate = [&](const uint32_t (&w)[WORDS]) {
                if constexpr (DT == ELX_F32) {
#pragma unroll
                    for (int i = 0; i < WORDS; ++i) acc[i] = fmaf(__uint_as_float(w[i]), inv_w, acc[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < WORDS; ++i) {
                        const float2 f = Lp<DT>::unpack2(w[i]);
                        acc[2 * i] = fmaf(f.x, inv_w, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(f.y, inv_w, acc[2 * i + 1]);
                    }
                }
            };
            if constexpr (kWorld > 0) {
                uint32_t raw[kWorld][WORDS];
#pragma unroll
                for (int j = 0; j < kWorld; ++j)
                    ld_words<WORDS>(static_cast<const char*>(a.grads.base[j]) + (src0 + mine) * Lp<DT>::kBytes, raw[j]);
                // keep every rank's words live until all loads are issued: the empty asm statements are ordered
                // after the (volatile) loads, so the compiler cannot fold a load into its first use
#pragma unroll
                for (int j = 0; j < kWorld; ++j) {
#pragma unroll
                    for (int i = 0; i < WORDS; i += 8)
                        asm volatile(""
                                     : "+r"(raw[j][i]), "+r"(raw[j][i + 1]), "+r"(raw[j][i + 2]), "+r"(raw[j][i + 3]),
                                       "+r"(raw[j][i + 4]), "+r"(raw[j][i + 5]), "+r"(raw[j][i + 6]), "+r"(raw[j][i + 7]));
                }
#pragma unroll
                for (int j = 0; j < kWorld; ++j) accumulate(raw[j]);    // rank order
            } else {
                for (int j = 0; j < world; ++j) {
                    uint32_t raw[WORDS];
                    ld_words<WORDS>(static_cast<const char*>(a.grads.base[j]) + (src0 + mine) * Lp<DT>::kBytes, raw);
                    accumulate(raw);
                }
            }
            uint32_t out[WORDS];
            if constexpr (DT == ELX_F32) {
#pragma unroll
                for (int i = 0; i < WORDS; ++i) out[i] = __float_as_uint(acc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < WORDS; ++i) out[i] = Lp<DT>::pack2(acc[2 * i], acc[2 * i + 1]);
            }
            st_words<WORDS>(static_cast<char*>(dst) + mine * Lp<DT>::kBytes, out);
            if (all_valid) {
#pragma unroll
                for (int i = 0; i < WORDS; ++i) bad |= Lp<DT>::nonfinite_word(out[i]);
            }
        } else {
            T* out = static_cast<T*>(dst);
            for (int64_t e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
                float acc = 0.0f;
                for (int j = 0; j < world; ++j)
                    acc = fmaf(Lp<DT>::to_float(static_cast<const T*>(a.grads.base[j])[src0 + e]), inv_w, acc);
                const T val = Lp<DT>::from_float(acc);
                out[e] = val;
                if (e < n_valid && Lp<DT>::nonfinite(val)) bad = 1;
            }
        }
        const unsigned any_bad = __ballot_sync(0xFFFFFFFFu, bad != 0);
        if (any_bad && lane == 0) {
            if (a.chunk_flags) atomicOr(&a.chunk_flags[s_cur.index], 1u);
            if (a.ctl) atomicOr(&a.ctl->found_inf, 1u);
        }
    }
    const unsigned ballot_desc = __ballot_sync(0xFFFFFFFFu, bad_desc);
    if (ballot_desc && lane == 0 && a.ctl) atomicOr(&a.ctl->status, ELX_STAT_BAD_DESC);
}

int grid_for(int64_t work_items, int ctas_per_sm);
int capped(int resident, int cap);

template <int DT, int kWorld>
int launch_pull_inst(const PullArgs& a, cudaStream_t s) {
    static const int resident = resident_ctas(pull_reduce_kernel<DT, kWorld>, 256);
    const int grid = grid_for(a.n_tiles, capped(resident, g_tune.pull_ctas_per_sm));
    if (grid < 0) return grid;
    pull_reduce_kernel<DT, kWorld><<<grid, 256, 0, s>>>(a);
    return record_cuda(cudaGetLastError());
}

template <int DT>
int launch_pull(const PullArgs& a, cudaStream_t s) {
    switch (a.grads.world) {
        case 2: return launch_pull_inst<DT, 2>(a, s);
        case 4: return launch_pull_inst<DT, 4>(a, s);
        case 8: return launch_pull_inst<DT, 8>(a, s);
    }
    return launch_pull_inst<DT, 0>(a, s);
}

// Flag region of one rank (peer-mapped): for each parity of the epoch and each sender, {epoch, word}.
// A rank can run at most one barrier ahead of a peer, so two parities are enough.
__device__ __forceinline__ uint32_t* flag_slot(void* region, uint32_t epoch, int sender) {
    return static_cast<uint32_t*>(region) + ((epoch & 1u) * ELX_MAX_PEERS + sender) * 2;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// One warp.  Lane j tells rank j "rank `rank` reached barrier `epoch`" (with this rank's overflow word
// riding along), then waits — for at most timeout_ns — until rank j has told this rank the same.
// On expiry the sticky ELX_STAT_TIMEOUT bit is raised and the kernel returns; it never traps.
__global__ void peer_barrier_kernel(ElxPeerTable flags, uint32_t epoch, ElxCtl* ctl, int exchange_overflow,
                                    uint64_t timeout_ns) {
    const int j = threadIdx.x;
    const int world = flags.world, rank = flags.rank;
    uint32_t seen_inf = 0;
    bool expired = false;
    if (j < world) {
        const uint32_t mine = (exchange_overflow && ctl) ? ctl->found_inf : 0u;
        __threadfence_system();   // everything this rank wrote before the barrier is visible to the peers first
        uint32_t* out = flag_slot(flags.base[j], epoch, rank);
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(out + 1), "r"(mine) : "memory");
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(out), "r"(epoch) : "memory");
        const uint32_t* in = flag_slot(flags.base[rank], epoch, j);
        const uint64_t t_start = global_timer_ns();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(in) : "memory");
            if (v == epoch) break;
            if (global_timer_ns() - t_start > timeout_ns) {
                expired = true;
                break;
            }
            __nanosleep(200);
        }
        if (!expired) asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(seen_inf) : "l"(in + 1) : "memory");
    }
    const unsigned any_inf = __ballot_sync(0xFFFFFFFFu, seen_inf != 0);
    const unsigned any_expired = __ballot_sync(0xFFFFFFFFu, expired);
    if (j == 0 && ctl) {
        if (exchange_overflow && any_inf) atomicOr(&ctl->found_inf, 1u);
        if (any_expired) atomicOr(&ctl->status, ELX_STAT_TIMEOUT);
    }
}

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

__global__ void step_begin_kernel(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const bool found = ctl->found_inf != 0;
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
                if (cfg.min_scale > 0.0f) scale = fmaxf(scale, cfg.min_scale);
            }
        }
    } else {
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
    }
    ctl->scale = scale;
    ctl->found_inf = 0;
}

// ------------------------------------------------------------------------------------------------
// launch helpers
// ------------------------------------------------------------------------------------------------

int grid_for(int64_t work_items, int ctas_per_sm) {
    const int sms = sm_count();
    if (sms < 0) return sms;
    int64_t g = static_cast<int64_t>(sms) * ctas_per_sm;
    if (g > work_items) g = work_items;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}

int capped(int resident, int cap) { return cap > 0 && cap < resident ? cap : resident; }

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

template <int DT, int MATH>
int launch_adam_tma(const AdamArgs& a, cudaStream_t s) {
    constexpr int smem = kTmaStages * TmaStage<DT>::kBytes;
    // the opt-in to more than 48 KB of dynamic shared memory is per device: once for each ordinal
    static bool opted_in[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    if (!opted_in[dev]) {
        const cudaError_t attr =
            cudaFuncSetAttribute(adam_tma_kernel<DT, MATH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (attr != cudaSuccess) {
            const int rc = record_cuda(attr);
            (void)cudaGetLastError();
            return rc;
        }
        opted_in[dev] = true;
    }
    const int grid = grid_for(a.n_tiles, 1);
    if (grid < 0) return grid;
    adam_tma_kernel<DT, MATH><<<grid, kTmaThreads, smem, s>>>(a);
    return record_cuda(cudaGetLastError());
}

template <int DT>
int launch_adam_dt(const AdamArgs& a, cudaStream_t s) {
    const bool precise = g_tune.math_mode == 1;
    if (g_tune.adam_variant == 1 || a.push.world > 0)
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

template <int DT, bool COPY, bool NORM, int UNROLL>
int launch_probe_inst(const ProbeArgs& a, cudaStream_t s) {
    static const int resident = resident_ctas(probe_kernel<DT, COPY, NORM, UNROLL>, kProbeThreads);
    const int64_t groups = (a.n_tiles + UNROLL - 1) / UNROLL;
    const int grid = grid_for(groups, capped(resident, g_tune.probe_ctas_per_sm));
    if (grid < 0) return grid;
    probe_kernel<DT, COPY, NORM, UNROLL><<<grid, kProbeThreads, 0, s>>>(a);
    return record_cuda(cudaGetLastError());
}

template <int DT, bool COPY>
int launch_probe_norm(const ProbeArgs& a, bool norm, cudaStream_t s) {
    // fp32 tiles are twice as many bytes: half the unroll keeps the register budget
    constexpr int kBig = DT == ELX_F32 ? 4 : 8;
    constexpr int kSmall = DT == ELX_F32 ? 2 : 4;
    const bool big = g_tune.probe_unroll >= 8;
    if (norm) return big ? launch_probe_inst<DT, COPY, true, kBig>(a, s) : launch_probe_inst<DT, COPY, true, kSmall>(a, s);
    return big ? launch_probe_inst<DT, COPY, false, kBig>(a, s) : launch_probe_inst<DT, COPY, false, kSmall>(a, s);
}

template <bool COPY>
int launch_probe(const ProbeArgs& a, int dtype, bool norm, cudaStream_t s) {
    switch (dtype) {
        case ELX_F16: return launch_probe_norm<ELX_F16, COPY>(a, norm, s);
        case ELX_BF16: return launch_probe_norm<ELX_BF16, COPY>(a, norm, s);
        case ELX_F32: return launch_probe_norm<ELX_F32, COPY>(a, norm, s);
    }
    return ELX_ERR_DTYPE;
}

int probe_single(const void* src, void* dst, int dtype, int64_t n_shard, int64_t n_valid, uint32_t* flag,
                 ElxCtl* ctl, float* l2sq, float* scratch, int64_t scratch_elems, void* stream, bool copy) {
    if (!src || (copy && !dst)) return ELX_ERR_NULL;
    if (!flag && !ctl && !l2sq && !copy) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (n_shard < 0 || n_valid < 0 || n_valid > n_shard) return ELX_ERR_SIZE;
    if (!aligned(src, 32) || (copy && !aligned(dst, 32))) return ELX_ERR_ALIGN;
    if ((flag && !aligned(flag, 4)) || (ctl && !aligned(ctl, 16)) || (l2sq && !aligned(l2sq, 4))) return ELX_ERR_ALIGN;
    if (copy) {
        const char* s0 = static_cast<const char*>(src);
        const char* d0 = static_cast<const char*>(dst);
        const int64_t bytes = n_shard * dtype_bytes(dtype);
        if (s0 < d0 + bytes && d0 < s0 + bytes) return ELX_ERR_ARG;
    }
    const int64_t n_tiles = (n_shard + kTile - 1) / kTile;
    if (l2sq) {
        if (!scratch) return ELX_ERR_NULL;
        if (!aligned(scratch, 4)) return ELX_ERR_ALIGN;
        if (scratch_elems < elx_probe_scratch_elems(n_tiles)) return ELX_ERR_SIZE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n_tiles == 0) {
        if (l2sq) return record_cuda(cudaMemsetAsync(l2sq, 0, sizeof(float), s));
        return ELX_OK;
    }
    ProbeArgs a;
    memset(&a, 0, sizeof(a));
    a.one_flag = flag;
    a.ctl = ctl;
    a.scratch = scratch;
    a.copy_dst = dst;
    a.first = 0;
    a.count = 1;
    a.inline_tables = 1;
    a.n_tiles = n_tiles;
    a.one_desc.grad_param = const_cast<void*>(src);
    a.one_desc.n_shard = n_shard;
    a.one_desc.n_valid = n_valid;
    a.one_desc.tile_begin = 0;
    a.one_desc.dtype = dtype;
    int rc = copy ? launch_probe<true>(a, dtype, l2sq != nullptr, s) : launch_probe<false>(a, dtype, l2sq != nullptr, s);
    if (rc != ELX_OK) return rc;
    if (l2sq) {
        NormArgs na;
        memset(&na, 0, sizeof(na));
        na.scratch = scratch;
        na.one_l2sq = l2sq;
        na.first = 0;
        na.count = 1;
        na.inline_tables = 1;
        na.one_desc = a.one_desc;
        norm_finalize<<<1, 256, 0, s>>>(na);
        rc = record_cuda(cudaGetLastError());
    }
    return rc;
}

// ------------------------------------------------------------------------------------------------
// built-in scratch for callers that cannot allocate
// ------------------------------------------------------------------------------------------------

// One partial sum per tile, so the largest shard elx_grad_check_static accepts has this many tiles
// (16384 tiles x 4096 elements = 67 108 864 elements).  64 KiB on every GPU that loads the library.
constexpr int64_t kStaticScratchTiles = 16384;
static __device__ __align__(256) float g_static_scratch[kStaticScratchTiles];

// Device address of g_static_scratch per device ordinal.  In host code the array's name is only a
// handle for the runtime, not something a kernel may dereference; the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
float* g_static_scratch_addr[64];

int static_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        if (e != cudaSuccess) record_cuda(e);
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    if (g_static_scratch_addr[dev] == nullptr) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_scratch);
        if (e != cudaSuccess || addr == nullptr) {
            record_cuda(e);
            (void)cudaGetLastError();
            return e == cudaSuccess ? ELX_ERR_NODEVICE : ELX_ERR_LAUNCH;
        }
        g_static_scratch_addr[dev] = static_cast<float*>(addr);
    }
    *out = g_static_scratch_addr[dev];
    return ELX_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------

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
        {"adam_min_blocks", &g_tune.adam_min_blocks, def.adam_min_blocks, 1, 3},
        {"adam_ctas_per_sm", &g_tune.adam_ctas_per_sm, def.adam_ctas_per_sm, 0, 32},
        {"probe_ctas_per_sm", &g_tune.probe_ctas_per_sm, def.probe_ctas_per_sm, 0, 32},
        {"probe_unroll", &g_tune.probe_unroll, def.probe_unroll, 4, 8},
        {"math_mode", &g_tune.math_mode, def.math_mode, 1, 2},
        {"adam_variant", &g_tune.adam_variant, def.adam_variant, 0, 1},
        {"pull_ctas_per_sm", &g_tune.pull_ctas_per_sm, def.pull_ctas_per_sm, 0, 32},
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
        *k.slot = value;
        return ELX_OK;
    }
    return ELX_ERR_ARG;
}

int64_t elx_probe_scratch_elems(int64_t n_tiles) { return n_tiles < 0 ? 0 : n_tiles; }

int elx_ctl_init(ElxCtl* ctl, float initial_scale, void* stream) {
    if (!ctl) return ELX_ERR_NULL;
    if (!aligned(ctl, 16)) return ELX_ERR_ALIGN;
    if (!(initial_scale > 0.0f)) return ELX_ERR_ARG;
    ctl_init_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctl, initial_scale);
    return record_cuda(cudaGetLastError());
}

int elx_step_begin(ElxCtl* ctl, ElxScalerCfg cfg, const float* norm_sq, void* stream) {
    if (!ctl) return ELX_ERR_NULL;
    if (!aligned(ctl, 16) || (norm_sq && !aligned(norm_sq, 4))) return ELX_ERR_ALIGN;
    if (cfg.dynamic) {
        if (!(cfg.growth_factor > 0.0f) || !(cfg.backoff_factor > 0.0f) || cfg.growth_interval <= 0 ||
            cfg.hysteresis < 0)
            return ELX_ERR_ARG;
    }
    if (cfg.max_norm > 0.0f && !norm_sq) return ELX_ERR_NULL;
    step_begin_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctl, cfg, norm_sq);
    return record_cuda(cudaGetLastError());
}

int elx_grad_check(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl, float* l2sq,
                   float* scratch, int64_t scratch_elems, void* stream) {
    return probe_single(g, nullptr, dtype, n_valid, n_valid, flag, ctl, l2sq, scratch, scratch_elems, stream, false);
}

int64_t elx_grad_check_static_max_elems(void) { return kStaticScratchTiles * kTile; }

int elx_grad_check_static(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl, float* l2sq,
                          void* stream) {
    if (n_valid > kStaticScratchTiles * kTile) return ELX_ERR_CAPACITY;
    float* scratch = nullptr;
    if (l2sq) {
        const int rc = static_scratch(&scratch);
        if (rc != ELX_OK) return rc;
    }
    return probe_single(g, nullptr, dtype, n_valid, n_valid, flag, ctl, l2sq, scratch, kStaticScratchTiles, stream,
                        false);
}

int elx_reduce_epilogue(const void* src, void* dst, int dtype, int64_t n_shard, int64_t n_valid, uint32_t* flag,
                        ElxCtl* ctl, float* l2sq, float* scratch, int64_t scratch_elems, void* stream) {
    return probe_single(src, dst, dtype, n_shard, n_valid, flag, ctl, l2sq, scratch, scratch_elems, stream, true);
}

int elx_grad_check_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                         uint32_t* chunk_flags, ElxCtl* ctl, float* chunk_l2sq, float* total_l2sq, float* scratch,
                         int64_t scratch_elems, void* stream) {
    if (!descs) return ELX_ERR_NULL;
    if (!chunk_flags && !ctl && !chunk_l2sq && !total_l2sq) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (first < 0 || count < 0 || n_tiles < 0) return ELX_ERR_SIZE;
    if (!aligned(descs, 8) || (chunk_flags && !aligned(chunk_flags, 4)) || (ctl && !aligned(ctl, 16)))
        return ELX_ERR_ALIGN;
    const bool norm = chunk_l2sq || total_l2sq;
    if (norm) {
        if (!scratch) return ELX_ERR_NULL;
        if (!aligned(scratch, 4)) return ELX_ERR_ALIGN;
        if (scratch_elems < elx_probe_scratch_elems(n_tiles)) return ELX_ERR_SIZE;
    }
    if (count == 0) return ELX_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = ELX_OK;
    if (n_tiles > 0) {
        ProbeArgs a;
        memset(&a, 0, sizeof(a));
        a.descs = descs;
        a.chunk_flags = chunk_flags;
        a.ctl = ctl;
        a.scratch = scratch;
        a.first = first;
        a.count = count;
        a.n_tiles = n_tiles;
        rc = launch_probe<false>(a, dtype, norm, s);
        if (rc != ELX_OK) return rc;
    }
    if (norm) {
        NormArgs na;
        memset(&na, 0, sizeof(na));
        na.descs = descs;
        na.scratch = scratch;
        na.chunk_l2sq = chunk_l2sq;
        na.total_l2sq = total_l2sq;
        na.first = first;
        na.count = count;
        norm_finalize<<<1, 256, 0, s>>>(na);
        rc = record_cuda(cudaGetLastError());
    }
    return rc;
}

int elx_adam_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype, const ElxSeg* segs,
                   const ElxHyper* hyper, int n_groups, ElxCtl* ctl, void* stream) {
    if (!descs || !ctl) return ELX_ERR_NULL;
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
    return launch_adam(a, dtype, static_cast<cudaStream_t>(stream));
}

static int peer_table_ok(const ElxPeerTable& t) {
    if (t.world < 1 || t.world > ELX_MAX_PEERS || t.rank < 0 || t.rank >= t.world) return ELX_ERR_SIZE;
    for (int j = 0; j < t.world; ++j) {
        if (!t.base[j]) return ELX_ERR_NULL;
        if (!aligned(t.base[j], 32)) return ELX_ERR_ALIGN;
    }
    return ELX_OK;
}

int elx_enable_peer_access(int peer_device) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        record_cuda(e);
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    if (peer_device == dev) return ELX_OK;
    int can = 0;
    e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
    if (e != cudaSuccess || !can) {
        if (e != cudaSuccess) record_cuda(e);
        (void)cudaGetLastError();
        return ELX_ERR_ARG;
    }
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        return ELX_OK;
    }
    return record_cuda(e);
}

int elx_peer_alloc(int64_t bytes, void** ptr, void* handle) {
    if (!ptr || !handle) return ELX_ERR_NULL;
    if (bytes <= 0) return ELX_ERR_SIZE;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
    if (e != cudaSuccess) {
        const int rc = record_cuda(e);
        (void)cudaGetLastError();
        return rc;
    }
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        const int rc = record_cuda(e);
        (void)cudaGetLastError();
        (void)cudaFree(p);
        return rc;
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return ELX_OK;
}

int elx_peer_free(void* ptr) {
    if (!ptr) return ELX_ERR_NULL;
    const cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) {
        const int rc = record_cuda(e);
        (void)cudaGetLastError();
        return rc;
    }
    return ELX_OK;
}

int elx_ipc_open(const void* handle, void** base) {
    if (!handle || !base) return ELX_ERR_NULL;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
    memcpy(&h, handle, sizeof(h));
    void* ptr = nullptr;
    // opened with the ACCESSING device current: the driver maps the exporter's memory for this device and
    // turns peer access on as needed
    const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        const int rc = record_cuda(e);
        (void)cudaGetLastError();
        return rc;
    }
    *base = ptr;
    return ELX_OK;
}

int elx_peek_u32(const void* device_ptr, uint32_t* value) {
    if (!device_ptr || !value) return ELX_ERR_NULL;
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, device_ptr);
    if (e != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
        if (e != cudaSuccess) record_cuda(e);
        (void)cudaGetLastError();
        return ELX_ERR_ARG;
    }
    e = cudaMemcpy(value, device_ptr, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        const int rc = record_cuda(e);
        (void)cudaGetLastError();
        return rc;
    }
    return ELX_OK;
}

int elx_ipc_close(void* base) {
    if (!base) return ELX_ERR_NULL;
    const cudaError_t e = cudaIpcCloseMemHandle(base);
    if (e != cudaSuccess) {
        const int rc = record_cuda(e);
        (void)cudaGetLastError();
        return rc;
    }
    return ELX_OK;
}

int elx_peer_barrier(ElxPeerTable flags, uint32_t epoch, ElxCtl* ctl, int exchange_overflow, int timeout_ms,
                     void* stream) {
    const int rc = peer_table_ok(flags);
    if (rc != ELX_OK) return rc;
    if (ctl && !aligned(ctl, 16)) return ELX_ERR_ALIGN;
    if (exchange_overflow && !ctl) return ELX_ERR_NULL;
    if (timeout_ms <= 0 || epoch == 0) return ELX_ERR_ARG;
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, epoch, ctl, exchange_overflow,
                                                                      static_cast<uint64_t>(timeout_ms) * 1000000ull);
    return record_cuda(cudaGetLastError());
}

int elx_pull_reduce_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                          ElxPeerTable grads, const int64_t* block_off, uint32_t* chunk_flags, ElxCtl* ctl,
                          void* stream) {
    if (!descs || !block_off) return ELX_ERR_NULL;
    if (!dtype_ok(dtype)) return ELX_ERR_DTYPE;
    if (first < 0 || count < 0 || n_tiles < 0) return ELX_ERR_SIZE;
    const int rc = peer_table_ok(grads);
    if (rc != ELX_OK) return rc;
    if (!aligned(descs, 8) || !aligned(block_off, 8) || (chunk_flags && !aligned(chunk_flags, 4)) ||
        (ctl && !aligned(ctl, 16)))
        return ELX_ERR_ALIGN;
    if (count == 0 || n_tiles == 0) return ELX_OK;
    PullArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = descs;
    a.chunk_flags = chunk_flags;
    a.ctl = ctl;
    a.grads = grads;
    a.block_off = block_off;
    a.first = first;
    a.count = count;
    a.n_tiles = n_tiles;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case ELX_F16: return launch_pull<ELX_F16>(a, s);
        case ELX_BF16: return launch_pull<ELX_BF16>(a, s);
        case ELX_F32: return launch_pull<ELX_F32>(a, s);
    }
    return ELX_ERR_DTYPE;
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
