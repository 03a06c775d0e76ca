// Part of the elixir_b200 CUDA library (C ABI: include/elixir_b200.h).  See elx_common.cuh for the
// overview of the kernels and of how the sources are divided.
#include "elx_common.cuh"

using namespace elx;

namespace {

// ------------------------------------------------------------------------------------------------
// NVLink: pull reduce-scatter fused with the probe, and the cross-rank barrier
// ------------------------------------------------------------------------------------------------
//
// Every rank keeps its replicated gradient blocks in a slab that all ranks of the box can address
// (peer-mapped memory).  Rank r produces its shard of a chunk by READING the r-th slice of that
// chunk's block from every rank with ordinary loads (its own slice from local HBM, W - 1 slices over
// NVLink), summing float(x) * (1/W) in rank order in fp32, rounding once to the chunk dtype, storing
// the shard and probing the rounded result for inf/nan in the same pass.  Two variants: per-lane 256-bit
// peer loads, and bulk copies (cp.async.bulk, never multicast) of whole slices into shared memory.

struct PullArgs {
    const ElxChunkDesc* descs;
    uint32_t* chunk_flags;
    ElxCtl* ctl;
    ElxPeerTable grads;
    const int64_t* block_off;   // per descriptor: element offset of the chunk's block inside the slabs
    const int64_t* stage_off;   // null, or per descriptor: element offset of this rank's slice inside the buffers
                                // of the OTHER ranks (they are local staging copies of that slice alone)
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
        const int64_t own0 = a.block_off[s_cur.index] + static_cast<int64_t>(rank) * n_shard;   // element offsets
        const int64_t stg0 = a.stage_off ? a.stage_off[s_cur.index] : own0;
        auto src0_of = [&](int j) { return j == rank ? own0 : stg0; };
        void* const dst = s_cur.d.grad_param;
        const bool all_valid = e0 + kTile <= n_valid, none_valid = e0 >= n_valid;
        uint32_t bad = 0;
        if ((e1 - e0 == kTile) && (all_valid || none_valid) && ((own0 | stg0) & 15) == 0 &&
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
                    ld_words<WORDS>(static_cast<const char*>(a.grads.base[j]) + (src0_of(j) + mine) * Lp<DT>::kBytes, raw[j]);
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
                    ld_words<WORDS>(static_cast<const char*>(a.grads.base[j]) + (src0_of(j) + mine) * Lp<DT>::kBytes, raw);
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
                    acc = fmaf(Lp<DT>::to_float(static_cast<const T*>(a.grads.base[j])[src0_of(j) + e]), inv_w, acc);
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

// Bulk-copy variant of the pull for 16-bit chunks and a compile-time group size: one elected thread
// fetches the W slices of a tile (W bulk loads of 8 KB, W - 1 of them from peer-mapped memory, never
// multicast) into a shared-memory stage two tiles ahead; the warps sum the slices out of shared memory
// in rank order, store the shard tile and probe it.  Larger NVLink requests than per-lane loads, and the
// link stays busy while a tile is being summed.
// Ring depth.  With one CTA on every SM three stages of W slices of 8 KB each are enough (a deeper ring measured
// slower there: 12 stages at W = 2 took 20.2 ms against 19.3 ms for the step's pull phase).  When the pull runs
// on a few SMs beside an update kernel ("pull_tma_ctas"), three stages keep only 24 KB of remote data in flight
// per SM, about 7 GB/s each; the deep ring fills the shared memory (192 KB: 12 stages at W = 2, 6 at W = 4).
template <int kWorld, bool kDeep>
struct PullRing {
    static constexpr int kStages = kDeep ? (kWorld == 2 ? 12 : kWorld == 4 ? 6 : 3) : 3;
};
constexpr int kPullThreads = 256;

struct PullSlot {
    void* dst;            // shard base
    int64_t e0, e1;       // tile range inside the shard
    int64_t own0, stg0;   // element offsets of the slice in the own slab / in the other ranks' buffers
    int64_t n_valid;
    int chunk;
    int kind;             // 1 = staged in shared memory, 2 = ragged (direct loads), 3 = bad descriptor
};

template <int DT, int kWorld, bool kDeep>
__global__ void __launch_bounds__(kPullThreads, 1) pull_reduce_tma_kernel(const __grid_constant__ PullArgs a) {
    static_assert(DT != ELX_F32, "the staged pull is for 16-bit chunks");
    constexpr int kPullStages = PullRing<kWorld, kDeep>::kStages;
    using T = typename Lp<DT>::T;
    constexpr int kSliceBytes = kTile * 2;
    constexpr int kStageBytes = kWorld * kSliceBytes;
    extern __shared__ __align__(128) unsigned char s_dyn[];
    __shared__ PullSlot s_slot[kPullStages];
    __shared__ __align__(8) uint64_t s_full[kPullStages];
    __shared__ int s_abort;

    const ElxChunkDesc* __restrict__ descs = a.descs;
    const int rank = a.grads.rank;
    const float inv_w = 1.0f / static_cast<float>(kWorld);
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kPullStages; ++s) mbar_init(&s_full[s], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t tile_lo = descs[a.first].tile_begin;
    const int64_t my_tiles = blockIdx.x < a.n_tiles ? (a.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // producer-side cursor (thread 0 only)
    int64_t pc_t0 = 0, pc_t1 = 0;
    int pc_index = -1;
    ElxChunkDesc pc_d;

    auto produce = [&](int64_t k) {
        const int s = static_cast<int>(k % kPullStages);
        const int64_t t = tile_lo + blockIdx.x + k * gridDim.x;
        PullSlot slot;
        slot.kind = 3;
        if (!(t >= pc_t0 && t < pc_t1)) {
            int lo = a.first, hi = a.first + a.count - 1;
            while (lo < hi) {
                int mid = (lo + hi + 1) >> 1;
                if (descs[mid].tile_begin <= t) lo = mid; else hi = mid - 1;
            }
            pc_d = descs[lo];
            pc_index = lo;
            pc_t0 = pc_d.tile_begin;
            pc_t1 = pc_t0 + tiles_of(pc_d.n_shard);
        }
        if (t >= pc_t0 && t < pc_t1 && pc_d.dtype == DT) {
            slot.dst = pc_d.grad_param;
            slot.e0 = (t - pc_t0) * kTile;
            slot.e1 = min(slot.e0 + kTile, pc_d.n_shard);
            slot.own0 = a.block_off[pc_index] + static_cast<int64_t>(rank) * pc_d.n_shard;
            slot.stg0 = a.stage_off ? a.stage_off[pc_index] : slot.own0;
            slot.n_valid = pc_d.n_valid;
            slot.chunk = pc_index;
            const bool whole = slot.e1 - slot.e0 == kTile;
            const bool uniform = slot.e0 + kTile <= pc_d.n_valid || slot.e0 >= pc_d.n_valid;
            const bool lined_up = ((slot.own0 | slot.stg0) & 15) == 0 && (reinterpret_cast<uintptr_t>(slot.dst) & 31u) == 0;
            slot.kind = (whole && uniform && lined_up) ? 1 : 2;
        }
        s_slot[s] = slot;
        if (slot.kind == 1) {
            unsigned char* base = s_dyn + static_cast<size_t>(s) * kStageBytes;
            mbar_arrive_expect_tx(&s_full[s], kStageBytes);
#pragma unroll
            for (int i = 0; i < kWorld; ++i) {
                // start with a different rank in every CTA so that the requests spread over all links at once
                const int j = (rank + 1 + i + static_cast<int>(blockIdx.x)) % kWorld;
                const int64_t src = (j == rank ? slot.own0 : slot.stg0) + slot.e0;
                bulk_g2s(base + j * kSliceBytes, static_cast<const char*>(a.grads.base[j]) + src * 2, kSliceBytes,
                         &s_full[s]);
            }
        } else {
            mbar_arrive(&s_full[s]);
        }
    };

    if (threadIdx.x == 0) {
        for (int64_t k = 0; k < my_tiles && k < kPullStages; ++k) produce(k);
    }

    bool bad_desc = false;
    int64_t k = 0;
    for (; k < my_tiles; ++k) {
        const int s = static_cast<int>(k % kPullStages);
        const uint32_t parity = static_cast<uint32_t>((k / kPullStages) & 1);
        if (!mbar_wait_bounded(&s_full[s], parity)) s_abort = 1;
        __syncthreads();
        if (s_abort) break;
        const PullSlot slot = s_slot[s];
        uint32_t bad = 0;
        if (slot.kind == 1) {
            const unsigned char* base = s_dyn + static_cast<size_t>(s) * kStageBytes;
            const bool probed = slot.e0 + kTile <= slot.n_valid;
            // a thread owns 2 x 8 consecutive elements, 2048 apart: conflict-free 128-bit shared reads
#pragma unroll
            for (int h = 0; h < kTile / (kPullThreads * 8); ++h) {
                const int e = h * (kPullThreads * 8) + threadIdx.x * 8;
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
                for (int j = 0; j < kWorld; ++j) {    // rank order
                    const uint4 w = *reinterpret_cast<const uint4*>(base + j * kSliceBytes + e * 2);
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = Lp<DT>::unpack2(ww[i]);
                        acc[2 * i] = fmaf(f.x, inv_w, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(f.y, inv_w, acc[2 * i + 1]);
                    }
                }
                U4 out;
#pragma unroll
                for (int i = 0; i < 4; ++i) out.x[i] = Lp<DT>::pack2(acc[2 * i], acc[2 * i + 1]);
                st128(static_cast<char*>(slot.dst) + (slot.e0 + e) * 2, out);
                if (probed) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) bad |= Lp<DT>::nonfinite_word(out.x[i]);
                }
            }
        } else if (slot.kind == 2) {
            T* out = static_cast<T*>(slot.dst);
            for (int64_t e = slot.e0 + threadIdx.x; e < slot.e1; e += blockDim.x) {
                float acc = 0.0f;
                for (int j = 0; j < kWorld; ++j)
                    acc = fmaf(Lp<DT>::to_float(static_cast<const T*>(a.grads.base[j])[(j == rank ? slot.own0 : slot.stg0) + e]),
                               inv_w, acc);
                const T val = Lp<DT>::from_float(acc);
                out[e] = val;
                if (e < slot.n_valid && Lp<DT>::nonfinite(val)) bad = 1;
            }
        } else {
            bad_desc = true;
        }
        const unsigned any_bad = __ballot_sync(0xFFFFFFFFu, bad != 0);
        if (any_bad && lane == 0) {
            if (a.chunk_flags) atomicOr(&a.chunk_flags[slot.chunk], 1u);
            if (a.ctl) atomicOr(&a.ctl->found_inf, 1u);
        }
        __syncthreads();   // the stage has been consumed by every warp
        if (threadIdx.x == 0 && k + kPullStages < my_tiles) produce(k + kPullStages);
    }
    if (threadIdx.x == 0 && s_abort) {
        // gave up on tile k: loads already issued for later tiles still target this CTA's shared memory
        for (int64_t j = k; j < my_tiles && j < k + kPullStages; ++j)
            (void)mbar_wait_bounded(&s_full[j % kPullStages], static_cast<uint32_t>((j / kPullStages) & 1));
        if (a.ctl) atomicOr(&a.ctl->status, ELX_STAT_TIMEOUT);
    }
    const unsigned ballot_desc = __ballot_sync(0xFFFFFFFFu, bad_desc);
    if (ballot_desc && lane == 0 && a.ctl) atomicOr(&a.ctl->status, ELX_STAT_BAD_DESC);
}

template <int DT, int kWorld, bool kDeep = false>
int launch_pull_tma(const PullArgs& a, cudaStream_t s) {
    if constexpr (DT == ELX_F32) {
        return ELX_ERR_DTYPE;
    } else {
        constexpr int smem = PullRing<kWorld, kDeep>::kStages * kWorld * kTile * 2;
        static bool opted_in[64];
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
            (void)cudaGetLastError();
            return ELX_ERR_NODEVICE;
        }
        if (!opted_in[dev]) {
            const cudaError_t attr = cudaFuncSetAttribute(pull_reduce_tma_kernel<DT, kWorld, kDeep>,
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
        if (g_tune.pull_tma_ctas > 0 && g_tune.pull_tma_ctas < grid) grid = g_tune.pull_tma_ctas;
        pull_reduce_tma_kernel<DT, kWorld, kDeep><<<grid, kPullThreads, smem, s>>>(a);
        return record_cuda(cudaGetLastError());
    }
}

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
    if (g_tune.pull_variant == 1 && DT != ELX_F32) {
        const bool deep = g_tune.pull_tma_ctas > 0;   // few CTAs: each one keeps more data in flight
        switch (a.grads.world) {
            case 2: return deep ? launch_pull_tma<DT, 2, true>(a, s) : launch_pull_tma<DT, 2>(a, s);
            case 4: return deep ? launch_pull_tma<DT, 4, true>(a, s) : launch_pull_tma<DT, 4>(a, s);
            case 8: return launch_pull_tma<DT, 8>(a, s);
        }
    }
    switch (a.grads.world) {
        case 2: return launch_pull_inst<DT, 2>(a, s);
        case 4: return launch_pull_inst<DT, 4>(a, s);
        case 8: return launch_pull_inst<DT, 8>(a, s);
    }
    return launch_pull_inst<DT, 0>(a, s);
}

// dst[i] = sum over the ranks of element i, as the NVLink switch forms it (16-bit elements, 16 bytes per access).
template <int DT>
__global__ void __launch_bounds__(512) multimem_reduce_kernel(const char* __restrict__ src_mc, char* __restrict__ dst,
                                                              int64_t n16) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
        U4 r;
        if constexpr (DT == ELX_BF16) {
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r.x[0]), "=r"(r.x[1]), "=r"(r.x[2]), "=r"(r.x[3]) : "l"(src_mc + i * 16) : "memory");
        } else {
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r.x[0]), "=r"(r.x[1]), "=r"(r.x[2]), "=r"(r.x[3]) : "l"(src_mc + i * 16) : "memory");
        }
        st128(dst + i * 16, r);
    }
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
// The word that rides along carries the overflow in bit 0 and "a wait of mine expired" in bit 1, so that a
// rank that gave up anywhere makes every rank skip the step (elx_step_begin skips while the bit is set).
__global__ void peer_barrier_kernel(ElxPeerTable flags, uint32_t epoch, ElxCtl* ctl, int exchange_overflow,
                                    uint64_t timeout_ns) {
    const int j = threadIdx.x;
    const int world = flags.world, rank = flags.rank;
    uint32_t seen_inf = 0;
    bool expired = false;
    if (j < world) {
        const uint32_t mine = (exchange_overflow && ctl)
                                  ? ((ctl->found_inf ? 1u : 0u) | ((ctl->status & ELX_STAT_TIMEOUT) ? 2u : 0u))
                                  : 0u;
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
    const unsigned any_inf = __ballot_sync(0xFFFFFFFFu, (seen_inf & 1u) != 0);
    const unsigned any_expired = __ballot_sync(0xFFFFFFFFu, expired || (seen_inf & 2u) != 0);
    if (j == 0 && ctl) {
        if (exchange_overflow && any_inf) atomicOr(&ctl->found_inf, 1u);
        if (any_expired) atomicOr(&ctl->status, ELX_STAT_TIMEOUT);
    }
}

}  // namespace

extern "C" {

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

int elx_multimem_reduce(const void* src_mc, void* dst, int dtype, int64_t n, void* stream) {
    if (!src_mc || !dst) return ELX_ERR_NULL;
    if (dtype != ELX_F16 && dtype != ELX_BF16) return ELX_ERR_DTYPE;
    if (n < 0 || (n & 7) != 0) return ELX_ERR_SIZE;
    if (!aligned(src_mc, 16) || !aligned(dst, 16)) return ELX_ERR_ALIGN;
    if (n == 0) return ELX_OK;
    const int64_t n16 = n / 8;
    const int grid = grid_for((n16 + 511) / 512, 2);
    if (grid < 0) return grid;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == ELX_F16)
        multimem_reduce_kernel<ELX_F16><<<grid, 512, 0, s>>>(static_cast<const char*>(src_mc), static_cast<char*>(dst), n16);
    else
        multimem_reduce_kernel<ELX_BF16><<<grid, 512, 0, s>>>(static_cast<const char*>(src_mc), static_cast<char*>(dst), n16);
    return record_cuda(cudaGetLastError());
}

int elx_copy_async(void* dst, const void* src, int64_t bytes, void* stream) {
    if (!dst || !src) return ELX_ERR_NULL;
    if (bytes < 0) return ELX_ERR_SIZE;
    if (bytes == 0) return ELX_OK;
    return record_cuda(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDefault,
                                       static_cast<cudaStream_t>(stream)));
}

int elx_pull_reduce_multi(const ElxChunkDesc* descs, int first, int count, int64_t n_tiles, int dtype,
                          ElxPeerTable grads, const int64_t* block_off, const int64_t* stage_off,
                          uint32_t* chunk_flags, ElxCtl* ctl, void* stream) {
    if (!descs || !block_off) return ELX_ERR_NULL;
    if (stage_off && !aligned(stage_off, 8)) return ELX_ERR_ALIGN;
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
    a.stage_off = stage_off;
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

}  // extern "C"
