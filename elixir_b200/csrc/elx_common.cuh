// Chunk-level mixed-precision optimizer step for B200 (sm_100a): what the translation units share.
//
// Everything in the library is HBM- or NVLink-bandwidth work: each element of a chunk shard is read
// once and written once from a persistent grid sized to the SM count.  No tensor-core use: the
// arithmetic intensity is ~0.4 flop/byte.
//
// Sources
//   elx_control.cu   library state (tuning knobs, error text), control block: ctl_init, step_begin
//                    (skip decision, combined divisor, loss-scaler update, step count)
//   elx_adam.cu      unscale + Adam/AdamW on fp32 master / exp_avg / exp_avg_sq + rounded low-precision
//                    copy-back: bulk-copy (TMA) pipelined kernel, direct kernel, copy-back alone;
//                    optional push all-gather to peer-mapped gather blocks
//   elx_probe.cu     inf/nan probe of the reduced low-precision gradients (optionally fused with the
//                    copy into the shard, optionally with a fixed-order sum of squares)
//   elx_peer.cu      NVLink: pull reduce-scatter fused with the probe, device-side barrier, IPC set-up
//
// Semantics follow hpcaitech/Elixir's ElixirOptimizer.step (elixir/wrapper/optimizer.py:192-220),
// Chunk.update_extra_reduce_info / optim_update (elixir/chunk/core/chunk.py:345-356, 403-415) and
// the multi-tensor Adam (with div_scale) and DynamicGradScaler of ColossalAI that Elixir calls.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "elixir_b200.h"

namespace elx {

constexpr int kTile = ELX_TILE;
constexpr int kMaxGroups = 64;
constexpr int kProbeThreads = 256;   // 16 elements per thread and tile

// ------------------------------------------------------------------------------------------------
// host-side state (defined in elx_control.cu)
// ------------------------------------------------------------------------------------------------

extern thread_local char t_cuda_err[256];

// Launch-shape knobs (elx_set_tuning).  A CTAs-per-SM cap of 0 means "as many as are resident".
struct Tuning {
    int adam_threads = 256;
    int adam_ctas_per_sm = 0;
    int probe_ctas_per_sm = 0;
    int probe_unroll = 4;
    int probe_variant = 1;        // single-array probe: 0 = loads, 1 = bulk-copy ring for long arrays, 2 = ring always
    int math_mode = 1;
    int adam_variant = 1;         // 0 = direct global accesses, 1 = bulk-copy (TMA) pipeline
    int pull_ctas_per_sm = 0;
    int pull_variant = 1;         // 0 = per-lane loads, 1 = bulk-copy staging (16-bit chunks, W in {2, 4, 8})
    int adam_tma_ctas = 0;        // grid of the bulk-copy update kernel, 0 = one CTA per SM
    int pull_tma_ctas = 0;        // grid of the bulk-copy pull kernel, 0 = one CTA per SM
    int adam_tma_stages = 0;      // ring depth of the bulk-copy update kernel: 0 = the deepest that fits, 3 = three
};
extern Tuning g_tune;

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

// Record a CUDA error text for elx_last_cuda_error; returns ELX_OK or ELX_ERR_LAUNCH.
int record_cuda(cudaError_t e);
// SM count of the current device, or a negative status.
int sm_count();
// Grid of a persistent kernel: min(work items, SMs x CTAs per SM), or a negative status.
int grid_for(int64_t work_items, int ctas_per_sm);
int capped(int resident, int cap);

inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline bool dtype_ok(int dt) { return dt == ELX_F16 || dt == ELX_BF16 || dt == ELX_F32; }
inline int dtype_bytes(int dt) { return dt == ELX_F32 ? 4 : 2; }

inline int peer_table_ok(const ElxPeerTable& t) {
    if (t.world < 1 || t.world > ELX_MAX_PEERS || t.rank < 0 || t.rank >= t.world) return ELX_ERR_SIZE;
    for (int j = 0; j < t.world; ++j) {
        if (!t.base[j]) return ELX_ERR_NULL;
        if (!aligned(t.base[j], 32)) return ELX_ERR_ALIGN;
    }
    return ELX_OK;
}

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
    int vec_ok;       // every pointer of the descriptor is 32-byte aligned
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
                                   reinterpret_cast<uintptr_t>(d.grad_param) | reinterpret_cast<uintptr_t>(d.grad_src);
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

// Where the kernels read the gradient of a shard: a separate source, or the low-precision shard itself.
__device__ __forceinline__ const void* grad_source(const ElxChunkDesc& d) { return d.grad_src ? d.grad_src : d.grad_param; }

// Index (relative to the chunk's first segment) of the last segment with begin <= e, or -1.
__device__ __forceinline__ int find_seg(const ElxSeg* __restrict__ segs, int n, int64_t e) {
    int lo = 0, hi = n;   // first segment with begin > e
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (segs[mid].begin <= e) lo = mid + 1; else hi = mid;
    }
    return lo - 1;
}

// No segment of the chunk intersects [e0, e1): nothing to update there, only the working copy to refresh.
__device__ __forceinline__ bool range_uncovered(const ElxSeg* __restrict__ segs, int n, int64_t e0, int64_t e1,
                                                int64_t n_valid) {
    if (e0 >= n_valid) return true;   // segments lie inside [0, n_valid)
    const int si = find_seg(segs, n, e1 - 1);
    return si < 0 || segs[si].end <= e0;
}


// ------------------------------------------------------------------------------------------------
// bulk asynchronous copies (the TMA unit's untiled form) and the mbarriers that track them
// ------------------------------------------------------------------------------------------------

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

}  // namespace elx
