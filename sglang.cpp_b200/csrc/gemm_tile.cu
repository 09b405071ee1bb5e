// y = x W^T for many rows (prefill batches, M > 256): a persistent tiled GEMM on the tcgen05
// tensor cores.  Bound by the tensor pipe, so the layout is chosen for MMA issue rate:
//   * output tiles of 128 tokens x 256 features; the 128-token block of x is the MMA "A" operand
//     (tokens run along the TMEM lanes), 256 rows of W are the "B" operand; one k-block of 64
//     elements is four 128x256x16 MMAs fed from a 48 KB shared-memory stage (4-stage TMA ring);
//   * one CTA per SM walks its tiles in a fixed order; two 256-column accumulators in TMEM
//     (all 512 columns) let the epilogue of tile i run under the MMAs of tile i+1;
//   * tiles are ordered in bands of 16 token blocks (2048 tokens): inside a band the feature
//     tile moves slowest, so the CTAs running at one time share a few W tiles and the band's x
//     stays in L2 while W streams past once per band;
//   * gated epilogue (gate_up projection + SwiGLU): the B operand is 128 gate rows followed by
//     the 128 matching up rows, so one thread holds gate[m][n] and up[m][n] in the same
//     accumulator and writes act(gate) * up for 128 features.
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"
#include "tensormap.cuh"

namespace b200 {
namespace {

constexpr int kTM = 128;      // tokens per tile (UMMA M)
constexpr int kTN = 256;      // W rows per tile (UMMA N)
constexpr int kBK = 64;       // bf16 elements per k-block (one 128-byte swizzle row)
constexpr int kStages = 4;
constexpr int kBand = 16;     // token blocks per band
constexpr int kThreads = 192; // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr uint32_t kABytes = kTM * kBK * 2;   // 16 KB
constexpr uint32_t kBBytes = kTN * kBK * 2;   // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;

struct TileParams {
    __nv_bfloat16* y;           // [M, n_out]
    const __nv_bfloat16* bias;  // [n_out] or NULL (plain epilogue only)
    int M;
    int n_out;          // output features (N, or N/2 with a gated epilogue)
    int up_row_offset;  // row of W where the "up" half starts (gated only)
    int kb_total;       // K / 64
    int epilogue;       // B200_EPILOGUE_*
    int m_tiles, n_tiles;
    int* status;
    // Grouped mode (expert GEMMs with many rows per expert): group g multiplies rows
    // [offsets[g], offsets[g] + counts[g]) of x by rows [g * w_rows_per_group, ...) of w; counts and
    // offsets live in device memory, so the tile list is built on the device by every CTA.
    const int32_t* group_counts;
    const int32_t* group_offsets;
    int num_groups;
    int w_rows_per_group;
};

constexpr int kMaxGroups = 256;

// Where a tile lives: first row of x / y, rows of it that belong to the tile, first feature, first
// row of the weights (of the "gate" half when gated).
struct TileAt {
    int row0, valid, n0, w_row0;
};

template <int EPI>
__device__ __forceinline__ float gated_act_tile(float g) {
    if (EPI == B200_EPILOGUE_SWIGLU) return __fdividef(g, 1.0f + __expf(-g));  // 2 ulp in fp32, far below the bf16 step
    if (EPI == B200_EPILOGUE_GEGLU_ERF) return 0.5f * g * (1.0f + erff(g * 0.70710678118654752f));
    return 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
}

// Tile t of the walk: bands of kBand token blocks, feature tile slowest inside a band.
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int& mt, int& ntile) {
    const int per_band = kBand * n_tiles;
    const int band = t / per_band;
    const int r = t - band * per_band;
    const int bm = min(kBand, m_tiles - band * kBand);
    ntile = r / bm;
    mt = band * kBand + (r - ntile * bm);
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
tile_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const TileParams p) {
    constexpr bool GATED = EPI != B200_EPILOGUE_NONE;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ __align__(8) uint64_t acc_full_bar[2];
    __shared__ __align__(8) uint64_t acc_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&acc_full_bar[a]), 1);
            mbar_init(smem_u32(&acc_empty_bar[a]), 4);  // one arrival per epilogue warp
        }
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmap_x);
        tma_prefetch_desc(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait_prior();

    __shared__ int s_first_tile[kMaxGroups + 1];   // grouped mode: first tile of every group
    __shared__ int s_cnt[kMaxGroups], s_off[kMaxGroups];
    const bool grouped = p.group_counts != nullptr;
    constexpr int kOutTile = GATED ? kTN / 2 : kTN;
    if (grouped) {
        for (int g = threadIdx.x; g < p.num_groups; g += kThreads) {
            s_cnt[g] = p.group_counts[g];
            s_off[g] = p.group_offsets[g];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = 0;
            for (int g = 0; g < p.num_groups; ++g) {
                s_first_tile[g] = run;
                run += ((max(s_cnt[g], 0) + kTM - 1) / kTM) * p.n_tiles;
            }
            s_first_tile[p.num_groups] = run;
        }
        __syncthreads();
    }
    const int total_tiles = grouped ? s_first_tile[p.num_groups] : p.m_tiles * p.n_tiles;
    auto locate = [&](int t) -> TileAt {
        TileAt a;
        if (!grouped) {
            int mt, ntile;
            tile_coords(t, p.m_tiles, p.n_tiles, mt, ntile);
            a.row0 = mt * kTM;
            a.valid = min(kTM, p.M - a.row0);
            a.n0 = ntile * kOutTile;
            a.w_row0 = 0;
            return a;
        }
        int lo = 0, hi = p.num_groups;   // largest g with s_first_tile[g] <= t
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_first_tile[mid] <= t) lo = mid; else hi = mid;
        }
        const int r = t - s_first_tile[lo];
        const int mtiles = (s_cnt[lo] + kTM - 1) / kTM;
        const int ntile = r / mtiles, mt = r - ntile * mtiles;   // token block fastest: neighbours share W
        a.row0 = s_off[lo] + mt * kTM;
        a.valid = min(kTM, s_cnt[lo] - mt * kTM);
        a.n0 = ntile * kOutTile;
        a.w_row0 = lo * p.w_rows_per_group;
        return a;
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool failed = false;
            for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
                const TileAt at = locate(t);
                const int m0 = at.row0;
                const int n0 = at.w_row0 + at.n0;
                for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages) {
                        const uint32_t par = static_cast<uint32_t>(it / kStages - 1) & 1u;
                        if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), par, p.status, 111)) {
                            failed = true;
                            break;
                        }
                    }
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    const uint32_t dst = smem_base + s * kStageBytes;
                    mbar_arrive_expect_tx(bar, kStageBytes);
                    tma_load_2d(dst, &tmap_x, kb * kBK, m0, bar);
                    if (GATED) {
                        tma_load_2d(dst + kABytes, &tmap_w, kb * kBK, n0, bar);
                        tma_load_2d(dst + kABytes + kBBytes / 2, &tmap_w, kb * kBK, p.up_row_offset + n0, bar);
                    } else {
                        tma_load_2d(dst + kABytes, &tmap_w, kb * kBK, n0, bar);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16_m128(kTN);
            int it = 0, tcount = 0;
            bool failed = false;
            for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x, ++tcount) {
                const int acc = tcount & 1;
                if (tcount >= 2) {
                    const uint32_t par = static_cast<uint32_t>((tcount >> 1) - 1) & 1u;
                    if (!mbar_wait_bounded(smem_u32(&acc_empty_bar[acc]), par, p.status, 112)) {
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                }
                const uint32_t d = tmem_base + static_cast<uint32_t>(acc * kTN);
                for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t par = static_cast<uint32_t>(it / kStages) & 1u;
                    if (!mbar_wait_bounded(smem_u32(&full_bar[s]), par, p.status, 113)) {
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a0 = smem_base + s * kStageBytes;
                    const uint32_t b0 = a0 + kABytes;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        tc_mma_bf16(d, kmajor_sw128_desc(a0 + k * 32), kmajor_sw128_desc(b0 + k * 32), idesc,
                                    (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(smem_u32(&empty_bar[s]));
                }
                if (failed) break;
                tc_commit(smem_u32(&acc_full_bar[acc]));
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int tcount = 0;
        bool failed = false;
        for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x, ++tcount) {
            const TileAt at = locate(t);
            const int acc = tcount & 1;
            const uint32_t par = static_cast<uint32_t>(tcount >> 1) & 1u;
            if (!mbar_wait_bounded(smem_u32(&acc_full_bar[acc]), par, p.status, 114)) {
                failed = true;
                break;
            }
            tc_fence_after();
            const int m_local = q * 32 + lane;
            const int m = at.row0 + m_local;
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * kTN);
            constexpr int kOutCols = kOutTile;
            const int n_base = at.n0;
            __nv_bfloat16* yrow = p.y + static_cast<int64_t>(m) * p.n_out;
#pragma unroll 1
            for (int c = 0; c < kOutCols / 32; ++c) {
                uint32_t g[32], u[32];
                tmem_ld_32x32b_x32(t0 + static_cast<uint32_t>(c * 32), g);
                if (GATED) tmem_ld_32x32b_x32(t0 + static_cast<uint32_t>(kTN / 2 + c * 32), u);
                tmem_ld_wait();
                const int n = n_base + c * 32;
                if (m_local < at.valid && n < p.n_out) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (GATED) {
                            const float gv = round_bf16(__uint_as_float(g[j]));
                            const float uv = round_bf16(__uint_as_float(u[j]));
                            v[j] = gated_act_tile<EPI>(gv) * uv;
                        } else {
                            v[j] = __uint_as_float(g[j]);
                        }
                    }
                    if (!GATED && p.bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n + j < p.n_out) v[j] += __bfloat162float(p.bias[n + j]);
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (n + j < p.n_out) {  // n_out is a multiple of 8: whole 16-byte groups
                            uint4 o;
                            o.x = pack_bf16(v[j], v[j + 1]);
                            o.y = pack_bf16(v[j + 2], v[j + 3]);
                            o.z = pack_bf16(v[j + 4], v[j + 5]);
                            o.w = pack_bf16(v[j + 6], v[j + 7]);
                            *reinterpret_cast<uint4*>(yrow + n + j) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[acc]));
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

int launch_tile_gemm(void* y, const void* x, const void* w, const void* bias, int M, int N, int K,
                     int64_t ldx, int epilogue, int* status, cudaStream_t stream) {
    const bool gated = epilogue != B200_EPILOGUE_NONE;
    const int n_out = gated ? N / 2 : N;
    TileParams p;
    p.y = static_cast<__nv_bfloat16*>(y);
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.M = M;
    p.n_out = n_out;
    p.up_row_offset = N / 2;
    p.kb_total = K / kBK;
    p.epilogue = epilogue;
    p.m_tiles = div_ceil(M, kTM);
    p.n_tiles = div_ceil(n_out, gated ? kTN / 2 : kTN);
    p.status = status;
    p.group_counts = nullptr;
    p.group_offsets = nullptr;
    p.num_groups = 0;
    p.w_rows_per_group = 0;

    CUtensorMap tmap_x, tmap_w;
    int err = cached_tmap(&tmap_x, x, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                          static_cast<uint64_t>(ldx) * 2, kBK, kTM);
    if (err != B200_OK) return err;
    err = cached_tmap(&tmap_w, w, static_cast<uint64_t>(K), static_cast<uint64_t>(N),
                      static_cast<uint64_t>(K) * 2, kBK, gated ? kTN / 2 : kTN);
    if (err != B200_OK) return err;

    const uint32_t smem_bytes = kStages * kStageBytes + 1024;
    const int tiles = p.m_tiles * p.n_tiles;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    void (*kernel)(CUtensorMap, CUtensorMap, TileParams) = tile_gemm_kernel<B200_EPILOGUE_NONE>;
    if (epilogue == B200_EPILOGUE_SWIGLU) kernel = tile_gemm_kernel<B200_EPILOGUE_SWIGLU>;
    if (epilogue == B200_EPILOGUE_GEGLU) kernel = tile_gemm_kernel<B200_EPILOGUE_GEGLU>;
    if (epilogue == B200_EPILOGUE_GEGLU_ERF) kernel = tile_gemm_kernel<B200_EPILOGUE_GEGLU_ERF>;
    B200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem_bytes)));
    B200_CHECK_CUDA(launch_kernel(kernel, dim3(grid), dim3(kThreads), smem_bytes, stream, dim3(1, 1, 1),
                                  tmap_x, tmap_w, p));
    return B200_OK;
}

// Grouped form (expert layers with many rows per expert): group g multiplies rows
// [offsets[g], offsets[g] + counts[g]) of x [total_rows, K] by w[g] ([N, K], groups stacked).
int launch_grouped_tile_gemm(void* y, const void* x, const void* w, const int32_t* counts,
                             const int32_t* offsets, int num_groups, int64_t total_rows, int N, int K,
                             int epilogue, int* status, cudaStream_t stream) {
    if (num_groups > kMaxGroups) {
        set_last_error("grouped GEMM: %d groups exceed %d", num_groups, kMaxGroups);
        return B200_ERR_UNSUPPORTED;
    }
    const bool gated = epilogue != B200_EPILOGUE_NONE;
    const int n_out = gated ? N / 2 : N;
    TileParams p;
    p.y = static_cast<__nv_bfloat16*>(y);
    p.bias = nullptr;
    p.M = static_cast<int>(total_rows);
    p.n_out = n_out;
    p.up_row_offset = N / 2;
    p.kb_total = K / kBK;
    p.epilogue = epilogue;
    p.m_tiles = 0;
    p.n_tiles = div_ceil(n_out, gated ? kTN / 2 : kTN);
    p.status = status;
    p.group_counts = counts;
    p.group_offsets = offsets;
    p.num_groups = num_groups;
    p.w_rows_per_group = N;
    CUtensorMap tmap_x, tmap_w;
    int err = cached_tmap(&tmap_x, x, static_cast<uint64_t>(K), static_cast<uint64_t>(total_rows),
                          static_cast<uint64_t>(K) * 2, kBK, kTM);
    if (err != B200_OK) return err;
    err = cached_tmap(&tmap_w, w, static_cast<uint64_t>(K), static_cast<uint64_t>(num_groups) * N,
                      static_cast<uint64_t>(K) * 2, kBK, gated ? kTN / 2 : kTN);
    if (err != B200_OK) return err;
    const uint32_t smem_bytes = kStages * kStageBytes + 1024;
    void (*kernel)(CUtensorMap, CUtensorMap, TileParams) = tile_gemm_kernel<B200_EPILOGUE_NONE>;
    if (epilogue == B200_EPILOGUE_SWIGLU) kernel = tile_gemm_kernel<B200_EPILOGUE_SWIGLU>;
    if (epilogue == B200_EPILOGUE_GEGLU) kernel = tile_gemm_kernel<B200_EPILOGUE_GEGLU>;
    if (epilogue == B200_EPILOGUE_GEGLU_ERF) kernel = tile_gemm_kernel<B200_EPILOGUE_GEGLU_ERF>;
    B200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem_bytes)));
    // the number of tiles is only known on the device: one persistent CTA per SM
    B200_CHECK_CUDA(launch_kernel(kernel, dim3(sm_count()), dim3(kThreads), smem_bytes, stream, dim3(1, 1, 1),
                                  tmap_x, tmap_w, p));
    return B200_OK;
}

}  // namespace b200
