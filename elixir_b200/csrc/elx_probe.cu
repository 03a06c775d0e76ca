// Part of the elixir_b200 CUDA library (C ABI: include/elixir_b200.h).  See elx_common.cuh for the
// overview of the kernels and of how the sources are divided.
#include <atomic>

#include "elx_common.cuh"

using namespace elx;

namespace {

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
            struct { const void* grad_param; int64_t n_shard, n_valid; } d = {grad_source(s_cur.d), s_cur.d.n_shard,
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
// probe of one long contiguous array through a bulk-copy ring
// ------------------------------------------------------------------------------------------------
//
// The load/store probe above keeps 96 KB per SM in flight (3 CTAs x 256 threads x 128 B) and its rate grows
// with the resident CTAs (1.8 / 3.5 / 4.9 TB/s for 1 / 2 / 3 CTAs per SM): it is bound by bytes in flight, and
// registers are what limits those.  Here ONE CTA per SM keeps a ring of 6 x 32 KB in shared memory filled by
// cp.async.bulk (no registers held by data in flight); the CTA tests each stage from shared memory.  Probe only:
// no copy, no norm.  The array must start on a 16-byte boundary; a last piece shorter than 16 bytes is read
// with plain loads.

constexpr int kBulkProbeStages = 6;
constexpr int kBulkProbeStageBytes = 32768;
constexpr int kBulkProbeSmem = kBulkProbeStages * kBulkProbeStageBytes;

struct BulkProbeArgs {
    const unsigned char* src;
    int64_t bytes;      // probed bytes (n_valid elements)
    uint32_t* flag;     // may be null
    ElxCtl* ctl;        // may be null
};

template <int DT>
__global__ void __launch_bounds__(kProbeThreads, 1) probe_bulk_kernel(const __grid_constant__ BulkProbeArgs a) {
    using T = typename Lp<DT>::T;
    constexpr int kVecPerThread = kBulkProbeStageBytes / (kProbeThreads * 16);   // 8
    extern __shared__ __align__(128) unsigned char s_dyn[];
    __shared__ __align__(8) uint64_t s_full[kBulkProbeStages];
    __shared__ int s_abort;

    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kBulkProbeStages; ++s) mbar_init(&s_full[s], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t n_units = (a.bytes + kBulkProbeStageBytes - 1) / kBulkProbeStageBytes;
    const int64_t my_units = blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    auto unit_offset = [&](int64_t k) { return (blockIdx.x + k * gridDim.x) * static_cast<int64_t>(kBulkProbeStageBytes); };
    auto unit_bytes = [&](int64_t k) {
        const int64_t rest = a.bytes - unit_offset(k);
        return static_cast<uint32_t>(rest < kBulkProbeStageBytes ? rest : kBulkProbeStageBytes);
    };
    auto produce = [&](int64_t k) {    // thread 0 only
        const int s = static_cast<int>(k % kBulkProbeStages);
        const uint32_t len16 = unit_bytes(k) & ~15u;
        if (len16) {
            mbar_arrive_expect_tx(&s_full[s], len16);
            bulk_g2s(s_dyn + static_cast<size_t>(s) * kBulkProbeStageBytes, a.src + unit_offset(k), len16, &s_full[s]);
        } else {
            mbar_arrive(&s_full[s]);
        }
    };

    if (threadIdx.x == 0) {
        for (int64_t k = 0; k < my_units && k < kBulkProbeStages; ++k) produce(k);
    }

    uint32_t bad = 0;
    int64_t k = 0;
    for (; k < my_units; ++k) {
        const int s = static_cast<int>(k % kBulkProbeStages);
        const uint32_t parity = static_cast<uint32_t>((k / kBulkProbeStages) & 1);
        if (!mbar_wait_bounded(&s_full[s], parity)) s_abort = 1;
        __syncthreads();
        if (s_abort) break;
        const unsigned char* base = s_dyn + static_cast<size_t>(s) * kBulkProbeStageBytes;
        const uint32_t len = unit_bytes(k);
        if (len == kBulkProbeStageBytes) {
            // consecutive threads read consecutive 16-byte pieces: conflict-free 128-bit shared reads
#pragma unroll
            for (int h = 0; h < kVecPerThread; ++h) {
                const uint4 w = *reinterpret_cast<const uint4*>(base + (h * kProbeThreads + threadIdx.x) * 16);
                bad |= Lp<DT>::nonfinite_word(w.x) | Lp<DT>::nonfinite_word(w.y) | Lp<DT>::nonfinite_word(w.z) |
                       Lp<DT>::nonfinite_word(w.w);
            }
        } else {
            const uint32_t len16 = len & ~15u;
            for (uint32_t off = threadIdx.x * 16; off < len16; off += kProbeThreads * 16) {
                const uint4 w = *reinterpret_cast<const uint4*>(base + off);
                bad |= Lp<DT>::nonfinite_word(w.x) | Lp<DT>::nonfinite_word(w.y) | Lp<DT>::nonfinite_word(w.z) |
                       Lp<DT>::nonfinite_word(w.w);
            }
            // the last elements, fewer than 16 bytes of them, straight from global memory
            const uint32_t tail_elems = (len - len16) / Lp<DT>::kBytes;
            if (threadIdx.x < tail_elems) {
                const T x = reinterpret_cast<const T*>(a.src + unit_offset(k) + len16)[threadIdx.x];
                if (Lp<DT>::nonfinite(x)) bad = 1;
            }
        }
        __syncthreads();   // the stage has been read by every warp
        if (threadIdx.x == 0 && k + kBulkProbeStages < my_units) produce(k + kBulkProbeStages);
    }
    const unsigned any_bad = __ballot_sync(0xFFFFFFFFu, bad != 0);
    if (any_bad && lane == 0) {
        if (a.flag) atomicOr(a.flag, 1u);
        if (a.ctl) atomicOr(&a.ctl->found_inf, 1u);
    }
    if (threadIdx.x == 0 && s_abort) {
        // gave up on unit k: loads already issued for later units still target this CTA's shared memory
        for (int64_t j = k; j < my_units && j < k + kBulkProbeStages; ++j)
            (void)mbar_wait_bounded(&s_full[j % kBulkProbeStages], static_cast<uint32_t>((j / kBulkProbeStages) & 1));
        if (a.ctl) atomicOr(&a.ctl->status, ELX_STAT_TIMEOUT);
        if (a.flag) atomicOr(a.flag, 1u);    // an array that was not read to the end does not count as clean
        if (a.ctl) atomicOr(&a.ctl->found_inf, 1u);
    }
}

template <int DT>
int launch_probe_bulk_inst(const BulkProbeArgs& a, cudaStream_t s) {
    static bool opted_in[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    if (!opted_in[dev]) {
        const cudaError_t attr =
            cudaFuncSetAttribute(probe_bulk_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkProbeSmem);
        if (attr != cudaSuccess) {
            const int rc = record_cuda(attr);
            (void)cudaGetLastError();
            return rc;
        }
        opted_in[dev] = true;
    }
    const int64_t n_units = (a.bytes + kBulkProbeStageBytes - 1) / kBulkProbeStageBytes;
    const int grid = grid_for(n_units, 1);
    if (grid < 0) return grid;
    probe_bulk_kernel<DT><<<grid, kProbeThreads, kBulkProbeSmem, s>>>(a);
    return record_cuda(cudaGetLastError());
}

int launch_probe_bulk(const BulkProbeArgs& a, int dtype, cudaStream_t s) {
    switch (dtype) {
        case ELX_F16: return launch_probe_bulk_inst<ELX_F16>(a, s);
        case ELX_BF16: return launch_probe_bulk_inst<ELX_BF16>(a, s);
        case ELX_F32: return launch_probe_bulk_inst<ELX_F32>(a, s);
    }
    return ELX_ERR_DTYPE;
}

// The same ring over a table of chunks (elx_grad_check_multi without a norm).  A stage holds kTilesPerStage
// consecutive tiles of the table's tile numbering.  Nearly every stage lies inside one chunk, below its valid_end
// and on a 16-byte boundary: it is fetched by ONE bulk copy and tested as a whole (the producer decides that with
// a few comparisons against its cached chunk).  The other stages (a chunk boundary, a ragged tail, a gradient
// source off the 16-byte boundary) are described tile by tile: the aligned part of each tile is staged by a copy of
// its own, the rest is read with plain loads.  Overflow words are raised per chunk.

struct RingTile {
    const unsigned char* src;   // first element of the tile in global memory
    uint32_t valid_bytes;       // bytes of the tile that are probed (up to valid_end)
    int chunk;                  // descriptor index, -1 = nothing to probe
    int staged;                 // 1: the first valid_bytes & ~15 bytes are in the stage
};

template <int DT>
__global__ void __launch_bounds__(kProbeThreads, 1) probe_ring_multi_kernel(const __grid_constant__ ProbeArgs a) {
    using T = typename Lp<DT>::T;
    constexpr int kTileBytes = kTile * Lp<DT>::kBytes;
    constexpr int kTilesPerStage = kBulkProbeStageBytes / kTileBytes;   // 4 (16-bit) or 2 (fp32)
    constexpr int kVecPerThread = kBulkProbeStageBytes / (kProbeThreads * 16);
    extern __shared__ __align__(128) unsigned char s_dyn[];
    __shared__ RingTile s_tile[kBulkProbeStages][kTilesPerStage];
    __shared__ int s_whole[kBulkProbeStages];    // >= 0: the stage is one piece of this chunk; -1: see s_tile
    __shared__ __align__(8) uint64_t s_full[kBulkProbeStages];
    __shared__ int s_abort;

    const ElxChunkDesc* __restrict__ descs = a.descs;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kBulkProbeStages; ++s) mbar_init(&s_full[s], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t tile_lo = descs[a.first].tile_begin;
    const int64_t n_units = (a.n_tiles + kTilesPerStage - 1) / kTilesPerStage;
    const int64_t my_units = blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // producer-side cache of the chunk the last tile fell into (thread 0 only), in scalars
    int64_t pc_t0 = 0, pc_t1 = 0;        // its tile range
    int64_t pc_full_t1 = 0;              // tiles [pc_t0, pc_full_t1) lie wholly below valid_end
    int64_t pc_n_valid = 0;
    const unsigned char* pc_base = nullptr;
    int pc_index = -1;
    bool pc_ok = false;                  // right dtype
    bool pc_aligned = false;             // gradient source on a 16-byte boundary
    bool bad_desc = false;

    auto locate = [&](int64_t t) {       // thread 0 only
        if (t >= pc_t0 && t < pc_t1) return;
        int lo = a.first, hi = a.first + a.count - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (descs[mid].tile_begin <= t) lo = mid; else hi = mid - 1;
        }
        const ElxChunkDesc d = descs[lo];
        pc_index = lo;
        pc_t0 = d.tile_begin;
        pc_t1 = pc_t0 + tiles_of(d.n_shard);
        pc_n_valid = d.n_valid;
        pc_full_t1 = pc_t0 + d.n_valid / kTile;
        pc_base = static_cast<const unsigned char*>(grad_source(d));
        pc_ok = d.dtype == DT;
        pc_aligned = (reinterpret_cast<uintptr_t>(pc_base) & 15u) == 0;
    };

    auto produce = [&](int64_t k) {    // thread 0 only
        const int s = static_cast<int>(k % kBulkProbeStages);
        const int64_t it0 = (blockIdx.x + k * gridDim.x) * static_cast<int64_t>(kTilesPerStage);
        const int64_t t0 = tile_lo + it0;
        unsigned char* stage = s_dyn + static_cast<size_t>(s) * kBulkProbeStageBytes;
        locate(t0);
        if (it0 + kTilesPerStage <= a.n_tiles && t0 >= pc_t0 && t0 + kTilesPerStage <= pc_full_t1 && pc_ok && pc_aligned) {
            s_whole[s] = pc_index;
            mbar_arrive_expect_tx(&s_full[s], kBulkProbeStageBytes);
            bulk_g2s(stage, pc_base + (t0 - pc_t0) * kTileBytes, kBulkProbeStageBytes, &s_full[s]);
            return;
        }
        s_whole[s] = -1;
        uint32_t tx = 0;
#pragma unroll
        for (int j = 0; j < kTilesPerStage; ++j) {
            RingTile rt = {nullptr, 0u, -1, 0};
            if (it0 + j < a.n_tiles) {
                const int64_t t = t0 + j;
                locate(t);
                if (t >= pc_t0 && t < pc_t1 && pc_ok) {
                    const int64_t e0 = (t - pc_t0) * kTile;
                    const int64_t valid = pc_n_valid - e0;
                    if (valid > 0) {
                        rt.src = pc_base + e0 * Lp<DT>::kBytes;
                        rt.valid_bytes = static_cast<uint32_t>((valid < kTile ? valid : kTile) * Lp<DT>::kBytes);
                        rt.chunk = pc_index;
                        rt.staged = pc_aligned && (rt.valid_bytes & ~15u) != 0;
                        if (rt.staged) tx += rt.valid_bytes & ~15u;
                    }
                } else {
                    bad_desc = true;
                }
            }
            s_tile[s][j] = rt;
        }
        if (tx) {
            mbar_arrive_expect_tx(&s_full[s], tx);
#pragma unroll
            for (int j = 0; j < kTilesPerStage; ++j) {
                const RingTile rt = s_tile[s][j];
                if (rt.staged) bulk_g2s(stage + j * kTileBytes, rt.src, rt.valid_bytes & ~15u, &s_full[s]);
            }
        } else {
            mbar_arrive(&s_full[s]);   // nothing to load: the phase completes at once and publishes the tiles
        }
    };

    if (threadIdx.x == 0) {
        for (int64_t k = 0; k < my_units && k < kBulkProbeStages; ++k) produce(k);
    }

    auto raise = [&](uint32_t bad, int chunk) {
        const unsigned any_bad = __ballot_sync(0xFFFFFFFFu, bad != 0);
        if (any_bad && lane == 0) {
            if (a.chunk_flags) atomicOr(&a.chunk_flags[chunk], 1u);
            if (a.ctl) atomicOr(&a.ctl->found_inf, 1u);
        }
    };

    int64_t k = 0;
    for (; k < my_units; ++k) {
        const int s = static_cast<int>(k % kBulkProbeStages);
        const uint32_t parity = static_cast<uint32_t>((k / kBulkProbeStages) & 1);
        if (!mbar_wait_bounded(&s_full[s], parity)) s_abort = 1;
        __syncthreads();
        if (s_abort) break;
        const unsigned char* stage = s_dyn + static_cast<size_t>(s) * kBulkProbeStageBytes;
        const int whole = s_whole[s];
        if (whole >= 0) {
            uint32_t bad = 0;
            // consecutive threads read consecutive 16-byte pieces: conflict-free 128-bit shared reads
#pragma unroll
            for (int h = 0; h < kVecPerThread; ++h) {
                const uint4 w = *reinterpret_cast<const uint4*>(stage + (h * kProbeThreads + threadIdx.x) * 16);
                bad |= Lp<DT>::nonfinite_word(w.x) | Lp<DT>::nonfinite_word(w.y) | Lp<DT>::nonfinite_word(w.z) |
                       Lp<DT>::nonfinite_word(w.w);
            }
            raise(bad, whole);
        } else {
            for (int j = 0; j < kTilesPerStage; ++j) {
                const RingTile rt = s_tile[s][j];
                if (rt.chunk < 0) continue;     // the same for every thread
                uint32_t bad = 0;
                uint32_t from_global = 0;       // byte offset from which the tile is read with plain loads
                if (rt.staged) {
                    const uint32_t len16 = rt.valid_bytes & ~15u;
                    for (uint32_t off = threadIdx.x * 16; off < len16; off += kProbeThreads * 16) {
                        const uint4 w = *reinterpret_cast<const uint4*>(stage + j * kTileBytes + off);
                        bad |= Lp<DT>::nonfinite_word(w.x) | Lp<DT>::nonfinite_word(w.y) | Lp<DT>::nonfinite_word(w.z) |
                               Lp<DT>::nonfinite_word(w.w);
                    }
                    from_global = len16;
                }
                const uint32_t n_rest = (rt.valid_bytes - from_global) / Lp<DT>::kBytes;
                const T* rest = reinterpret_cast<const T*>(rt.src + from_global);
                for (uint32_t e = threadIdx.x; e < n_rest; e += kProbeThreads)
                    if (Lp<DT>::nonfinite(rest[e])) bad = 1;
                raise(bad, rt.chunk);
            }
        }
        __syncthreads();   // the stage and its records have been read by every warp
        if (threadIdx.x == 0 && k + kBulkProbeStages < my_units) produce(k + kBulkProbeStages);
    }
    if (threadIdx.x == 0) {
        if (s_abort) {
            for (int64_t j = k; j < my_units && j < k + kBulkProbeStages; ++j)
                (void)mbar_wait_bounded(&s_full[j % kBulkProbeStages], static_cast<uint32_t>((j / kBulkProbeStages) & 1));
            // chunks that were not read to the end do not count as clean
            if (a.ctl) {
                atomicOr(&a.ctl->status, ELX_STAT_TIMEOUT);
                atomicOr(&a.ctl->found_inf, 1u);
            }
            if (a.chunk_flags)
                for (int i = 0; i < a.count; ++i) atomicOr(&a.chunk_flags[a.first + i], 1u);
        }
        if (bad_desc && a.ctl) atomicOr(&a.ctl->status, ELX_STAT_BAD_DESC);
    }
}

template <int DT>
int launch_probe_ring_multi_inst(const ProbeArgs& a, cudaStream_t s) {
    static bool opted_in[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    if (!opted_in[dev]) {
        const cudaError_t attr = cudaFuncSetAttribute(probe_ring_multi_kernel<DT>,
                                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkProbeSmem);
        if (attr != cudaSuccess) {
            const int rc = record_cuda(attr);
            (void)cudaGetLastError();
            return rc;
        }
        opted_in[dev] = true;
    }
    constexpr int kTilesPerStage = kBulkProbeStageBytes / (kTile * Lp<DT>::kBytes);
    const int grid = grid_for((a.n_tiles + kTilesPerStage - 1) / kTilesPerStage, 1);
    if (grid < 0) return grid;
    probe_ring_multi_kernel<DT><<<grid, kProbeThreads, kBulkProbeSmem, s>>>(a);
    return record_cuda(cudaGetLastError());
}

int launch_probe_ring_multi(const ProbeArgs& a, int dtype, cudaStream_t s) {
    switch (dtype) {
        case ELX_F16: return launch_probe_ring_multi_inst<ELX_F16>(a, s);
        case ELX_BF16: return launch_probe_ring_multi_inst<ELX_BF16>(a, s);
        case ELX_F32: return launch_probe_ring_multi_inst<ELX_F32>(a, s);
    }
    return ELX_ERR_DTYPE;
}

// Arrays from this size on take the bulk-copy probe (probe_variant 1); below it the ring's ramp-up and drain
// outweigh what it gains.  probe_variant 2 sends every eligible array there (tests), 0 none.
constexpr int64_t kBulkProbeMinBytes = int64_t(16) << 20;

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
    // fp32 tiles are twice as many bytes: half the unroll keeps the register count
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
    // element alignment is enough: tiles whose addresses are not 32-byte aligned take the scalar path
    if (!aligned(src, dtype_bytes(dtype)) || (copy && !aligned(dst, dtype_bytes(dtype)))) return ELX_ERR_ALIGN;
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
    if (!copy && !l2sq && n_valid > 0 && aligned(src, 16) && g_tune.probe_variant != 0 &&
        (g_tune.probe_variant == 2 || n_valid * dtype_bytes(dtype) >= kBulkProbeMinBytes)) {
        BulkProbeArgs b;
        b.src = static_cast<const unsigned char*>(src);
        b.bytes = n_valid * dtype_bytes(dtype);
        b.flag = flag;
        b.ctl = ctl;
        return launch_probe_bulk(b, dtype, s);
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
// fp32 gradient reduction: widen before the collective, narrow + land + probe after it
// ------------------------------------------------------------------------------------------------

// dst[i] = float(src[i]).  16 elements per thread and tile, whole-line warp accesses; scalar tail.
template <int DT>
__global__ void __launch_bounds__(kProbeThreads) widen_kernel(const void* __restrict__ src, float* __restrict__ dst,
                                                              int64_t n, int vec_ok) {
    constexpr int EPT = kTile / kProbeThreads;
    const int64_t n_full = vec_ok ? n / kTile : 0;
    for (int64_t t = blockIdx.x; t < n_full; t += gridDim.x) {
        float g[EPT];
        load_lowp<DT, EPT>(src, t * kTile, g);
        store_f32<EPT>(dst, t * kTile, g);
    }
    const typename Lp<DT>::T* in = static_cast<const typename Lp<DT>::T*>(src);
    for (int64_t e = n_full * kTile + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < n;
         e += static_cast<int64_t>(gridDim.x) * blockDim.x)
        dst[e] = Lp<DT>::to_float(in[e]);
}

// dst[i] = round_to_nearest_even(src[i]) for i in [0, n_shard); the rounded values of [0, n_valid) are probed.
template <int DT>
__global__ void __launch_bounds__(kProbeThreads) narrow_probe_kernel(const float* __restrict__ src, void* dst,
                                                                     int64_t n_shard, int64_t n_valid, uint32_t* flag,
                                                                     ElxCtl* ctl, int vec_ok) {
    constexpr int EPT = kTile / kProbeThreads;
    using T = typename Lp<DT>::T;
    const int64_t n_full = vec_ok ? n_shard / kTile : 0;
    uint32_t bad = 0;
    for (int64_t t = blockIdx.x; t < n_full; t += gridDim.x) {
        float p[EPT];
        load_f32<EPT>(src, t * kTile, p);
        store_lowp<DT, EPT>(dst, t * kTile, p);
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int64_t e = t * kTile + group_offset<EPT>(j / 8) + (j & 7);
            if (e < n_valid && Lp<DT>::nonfinite(Lp<DT>::from_float(p[j]))) bad = 1;
        }
    }
    T* out = static_cast<T*>(dst);
    for (int64_t e = n_full * kTile + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < n_shard;
         e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const T val = Lp<DT>::from_float(src[e]);
        out[e] = val;
        if (e < n_valid && Lp<DT>::nonfinite(val)) bad = 1;
    }
    const unsigned any_bad = __ballot_sync(0xFFFFFFFFu, bad != 0);
    if (any_bad && (threadIdx.x & 31) == 0) {
        if (flag) atomicOr(flag, 1u);
        if (ctl) atomicOr(&ctl->found_inf, 1u);
    }
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
// cudaGetSymbolAddress, asked once per device with that device current.  Atomic: several host threads
// may make the first call on a device at once (they all store the same value).
std::atomic<float*> g_static_scratch_addr[64];

int static_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        if (e != cudaSuccess) record_cuda(e);
        (void)cudaGetLastError();
        return ELX_ERR_NODEVICE;
    }
    float* cached = g_static_scratch_addr[dev].load(std::memory_order_acquire);
    if (cached == nullptr) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_scratch);
        if (e != cudaSuccess || addr == nullptr) {
            record_cuda(e);
            (void)cudaGetLastError();
            return e == cudaSuccess ? ELX_ERR_NODEVICE : ELX_ERR_LAUNCH;
        }
        cached = static_cast<float*>(addr);
        g_static_scratch_addr[dev].store(cached, std::memory_order_release);
    }
    *out = cached;
    return ELX_OK;
}

}  // namespace

extern "C" {

int64_t elx_probe_scratch_elems(int64_t n_tiles) { return n_tiles < 0 ? 0 : n_tiles; }

int elx_grad_check(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl, float* l2sq,
                   float* scratch, int64_t scratch_elems, void* stream) {
    return probe_single(g, nullptr, dtype, n_valid, n_valid, flag, ctl, l2sq, scratch, scratch_elems, stream, false);
}

int64_t elx_grad_check_static_max_elems(void) { return kStaticScratchTiles * kTile; }

int elx_grad_check_static(const void* g, int dtype, int64_t n_valid, uint32_t* flag, ElxCtl* ctl, float* l2sq,
                          void* stream) {
    float* scratch = nullptr;
    if (l2sq) {
        // only the sum of squares uses the built-in array; the plain probe needs no scratch at any size
        if (g && dtype_ok(dtype) && n_valid > kStaticScratchTiles * kTile) return ELX_ERR_CAPACITY;
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

int elx_widen(const void* src, int dtype, float* dst, int64_t n, void* stream) {
    if (!src || !dst) return ELX_ERR_NULL;
    if (dtype != ELX_F16 && dtype != ELX_BF16) return ELX_ERR_DTYPE;
    if (n < 0) return ELX_ERR_SIZE;
    if (!aligned(src, 2) || !aligned(dst, 4)) return ELX_ERR_ALIGN;
    if (n == 0) return ELX_OK;
    const int vec_ok = aligned(src, 32) && aligned(dst, 32);
    const int grid = grid_for((n + kTile - 1) / kTile, 8);
    if (grid < 0) return grid;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == ELX_F16) widen_kernel<ELX_F16><<<grid, kProbeThreads, 0, s>>>(src, dst, n, vec_ok);
    else widen_kernel<ELX_BF16><<<grid, kProbeThreads, 0, s>>>(src, dst, n, vec_ok);
    return record_cuda(cudaGetLastError());
}

int elx_narrow_epilogue(const float* src, void* dst, int dtype, int64_t n_shard, int64_t n_valid, uint32_t* flag,
                        ElxCtl* ctl, void* stream) {
    if (!src || !dst) return ELX_ERR_NULL;
    if (dtype != ELX_F16 && dtype != ELX_BF16) return ELX_ERR_DTYPE;
    if (n_shard < 0 || n_valid < 0 || n_valid > n_shard) return ELX_ERR_SIZE;
    if (!aligned(src, 4) || !aligned(dst, 2) || (flag && !aligned(flag, 4)) || (ctl && !aligned(ctl, 16)))
        return ELX_ERR_ALIGN;
    if (n_shard == 0) return ELX_OK;
    const int vec_ok = aligned(src, 32) && aligned(dst, 32);
    const int grid = grid_for((n_shard + kTile - 1) / kTile, 8);
    if (grid < 0) return grid;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == ELX_F16)
        narrow_probe_kernel<ELX_F16><<<grid, kProbeThreads, 0, s>>>(src, dst, n_shard, n_valid, flag, ctl, vec_ok);
    else
        narrow_probe_kernel<ELX_BF16><<<grid, kProbeThreads, 0, s>>>(src, dst, n_shard, n_valid, flag, ctl, vec_ok);
    return record_cuda(cudaGetLastError());
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
        // without a norm: the bulk-copy ring from 16 MiB of tiles on (probe_variant 2: always, 0: never)
        const bool ring = !norm && g_tune.probe_variant != 0 &&
                          (g_tune.probe_variant == 2 || n_tiles * kTile * dtype_bytes(dtype) >= kBulkProbeMinBytes);
        rc = ring ? launch_probe_ring_multi(a, dtype, s) : launch_probe<false>(a, dtype, norm, s);
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

}  // extern "C"
