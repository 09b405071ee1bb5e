// All-reduce over NVLink peer memory (a one-shot kernel, and a two-shot kernel for groups of eight),
// alone or fused with the residual add + RMSNorm that follows every row-parallel projection under
// tensor parallelism.
//
// Stands where tensor_model_parallel_all_reduce does (src/distributed/distributed.cc:205-226,
// called from LinearRowParallel / LinearOProj::forward, src/layers/linear.cc:52-55,73-76), and
// folds in the RMSNorm::fused_add_forward_inplace the models run next.  One process per GPU.
//
//   * every rank owns two exchange buffers (call parity) and a flag table in ordinary device
//     memory; peers map them through CUDA IPC handles exchanged on the host;
//   * the producer GEMM writes its partial result straight into the local exchange buffer;
//   * the kernel announces "call c ready" to every peer (a store into the peer's flag table,
//     one slot per CTA so CTAs never coordinate), waits — bounded — for the same announcement
//     from every peer, then reads the peers' partials with plain uncached 16-byte loads (no
//     TMA), sums in fp32 in rank order, rounds to bf16 (the value the reference's all-reduce
//     returns) and continues with the add + norm on the row;
//   * call parity makes the buffers safe to reuse with this single barrier: a rank can only
//     start writing parity p again after a call in which every peer reported having finished
//     its previous read of parity p.
#include <mutex>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCommBlocks = 1024;  // CTAs per launch that take part in the handshake

struct CommDevice {
    const __nv_bfloat16* peer_buf[2][kMaxRanks];  // [parity][rank] -> that rank's exchange buffer
    uint32_t* peer_flags[kMaxRanks];              // [rank] -> that rank's flag table [blocks][ranks]
    uint32_t* self_counter;                       // [blocks] calls this CTA slot has completed
    void* peer_gather[kMaxRanks];                 // [rank] -> that rank's buffer of reduced rows (two-shot):
                                                  // 8-byte words of two bf16 values + the call number
    // NVLink multicast (NVLS) addresses of the same memory on every rank, or NULL: a load-reduce through
    // them is summed inside the switch, a store through them lands on every rank.
    const uint8_t* mc_buf[2];
    uint8_t* mc_gather;
    int rank, world;
    uint64_t wait_limit_ns;                       // longest a CTA waits for its peers before it gives up
};

// The poll side of every flag: an acquire load at system scope, so the data loads that follow the
// poll loop (after the CTA barrier) are ordered behind the flag they wait for.
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Handshake of one CTA slot with the same slot on every peer.  Returns false on time-out.
__device__ __forceinline__ bool comm_barrier(const CommDevice& c, int* status) {
    __shared__ int s_ok;
    const int slot = blockIdx.x % kMaxCommBlocks;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < c.world) {
        const uint32_t call = c.self_counter[slot] + 1;
        const int peer = threadIdx.x;
        // This rank's partial was written by the kernel before this one; make it visible to
        // the other GPUs before the flag that announces it.
        // No fence is needed before the flag store.  What it announces was written by the kernel
        // BEFORE this one, so it has been performed at this GPU's L2 (the point the peers read
        // from) before this kernel started; the peers poll with an acquire load and read the data
        // with uncached loads issued after their poll loop exits; and the loads of this rank's
        // previous call finished before that kernel ended, so a peer that sees the new flag may
        // overwrite the other parity's buffer.  (Measured on 2 x B200: 9 us per call with
        // fence.sys + st.release, 2 us with the relaxed store.)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(c.peer_flags[peer] + slot * kMaxRanks + c.rank),
                     "r"(call)
                     : "memory");
        const uint32_t* mine = c.peer_flags[c.rank] + slot * kMaxRanks + peer;
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(mine) - call) < 0) {
            if ((++spins & 0xffu) == 0 && global_timer_ns() - t0 > c.wait_limit_ns) {
                atomicExch(&status[kStatusTimeout], 401);
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) c.self_counter[slot] += 1;
    return s_ok != 0;
}

constexpr int kArVecPerThread = 4;  // 16-byte vectors a thread keeps in registers (hidden <= 8192)

// One CTA per row (grid-stride over rows).
// MODE 0: out = bf16(sum of partials)                       (tensor_model_parallel_all_reduce)
// MODE 1: residual <- bf16(sum) + residual; out <- rmsnorm  (+ RMSNorm::fused_add_forward_inplace)
template <int MODE, bool ROUND_FIRST>
__global__ void __launch_bounds__(256)
allreduce_kernel(const CommDevice c, int parity, __nv_bfloat16* out, __nv_bfloat16* residual,
                 const __nv_bfloat16* __restrict__ weight, int rows, int hidden, float eps, int* status) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait_prior();
    // A peer that never announced: leave `residual` and `out` as they are and let the host read
    // the status word (site 401).
    if (!comm_barrier(c, status)) return;
    const int nvec = hidden >> 3;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int64_t base = static_cast<int64_t>(row) * nvec;
        float vals[kArVecPerThread][8];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kArVecPerThread; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v >= nvec) continue;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < c.world; ++r) {  // rank order: every rank gets the same bits
                const uint4 a = __ldcv(reinterpret_cast<const uint4*>(c.peer_buf[parity][r]) + base + v);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[2 * j] += bf16_lo(aw[j]);
                    acc[2 * j + 1] += bf16_hi(aw[j]);
                }
            }
            uint32_t y[4];  // what the reference's all-reduce returns: the sum in bf16
#pragma unroll
            for (int j = 0; j < 4; ++j) y[j] = pack_bf16(acc[2 * j], acc[2 * j + 1]);
            if (MODE == 0) {
                reinterpret_cast<uint4*>(out)[base + v] = make_uint4(y[0], y[1], y[2], y[3]);
            } else {
                const uint4 rr = reinterpret_cast<const uint4*>(residual)[base + v];
                const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = bf16_lo(y[j]) + bf16_lo(rw[j]);
                    const float hi = bf16_hi(y[j]) + bf16_hi(rw[j]);
                    packed[j] = pack_bf16(lo, hi);
                    vals[i][2 * j] = ROUND_FIRST ? bf16_lo(packed[j]) : lo;
                    vals[i][2 * j + 1] = ROUND_FIRST ? bf16_hi(packed[j]) : hi;
                }
                reinterpret_cast<uint4*>(residual)[base + v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
            }
        }
        if (MODE == 0) continue;
        ss = warp_sum(ss);
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
        tot = warp_sum(tot);
        const float scale = rsqrtf(tot / static_cast<float>(hidden) + eps);
#pragma unroll
        for (int i = 0; i < kArVecPerThread; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v >= nvec) continue;
            const uint4 w4 = reinterpret_cast<const uint4*>(weight)[v];
            const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                o[j] = pack_bf16(vals[i][2 * j] * scale * bf16_lo(ww[j]), vals[i][2 * j + 1] * scale * bf16_hi(ww[j]));
            reinterpret_cast<uint4*>(out)[base + v] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}


// Two-shot variant: row `row` is reduced by rank row % world alone, which reads that row of every
// rank's partial (1/world of what the one-shot kernel reads) and pushes the bf16 sum into every
// peer's gather buffer.  Every rank then runs the same add + norm on the same bits, so the
// replicated residual stays replicated.  One CTA per row, grid = rows on every rank.
//   flag A (peer_flags of the owner, slot = row, one word per source rank): "my partial is written".
//   The pushed row needs no flag of its own and no fence: every 8-byte word of the gather buffer
//   holds two bf16 values and the call number, is written with one store and is polled by the
//   thread that consumes it (the low-latency protocol of collective libraries: half the link
//   bandwidth for one NVLink traversal instead of data + fence + flag + fetch).
// The gather buffer needs no parity: a rank can only reach this call's push of a row after every
// peer announced this call's partial, which each does after consuming the call before; words of
// earlier calls carry earlier numbers.
template <int MODE, bool ROUND_FIRST>
__global__ void __launch_bounds__(256)
allreduce_twoshot_kernel(const CommDevice c, int parity, __nv_bfloat16* out, __nv_bfloat16* residual,
                         const __nv_bfloat16* __restrict__ weight, int rows, int hidden, float eps, int* status) {
    __shared__ float red[32];
    __shared__ int s_ok;
    pdl_launch_dependents();
    pdl_wait_prior();
    const int row = blockIdx.x;          // also the flag slot
    const int owner = row % c.world;
    const uint32_t call = c.self_counter[row] + 1;
    const int nvec = hidden >> 3;
    const int64_t base = static_cast<int64_t>(row) * nvec;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    // announce this rank's partial to the row's owner (see comm_barrier for why a relaxed store is enough)
    if (threadIdx.x == 0)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(c.peer_flags[owner] + row * kMaxRanks + c.rank),
                     "r"(call)
                     : "memory");
    uint32_t y[kArVecPerThread][4];   // the bf16 sum of this thread's vectors
    if (c.rank == owner) {
        if (threadIdx.x < c.world) {
            const uint32_t* f = c.peer_flags[c.rank] + row * kMaxRanks + threadIdx.x;
            const uint64_t t0 = global_timer_ns();
            uint32_t spins = 0;
            while (static_cast<int32_t>(ld_acquire_sys(f) - call) < 0) {
                if ((++spins & 0xffu) == 0 && global_timer_ns() - t0 > c.wait_limit_ns) {
                    atomicExch(&status[kStatusTimeout], 402);
                    s_ok = 0;
                    break;
                }
            }
        }
        __syncthreads();
        // a partial never arrived: push nothing (the peers then run into their own limit, site 403)
        if (!s_ok) {
            if (threadIdx.x == 0) c.self_counter[row] = call;
            return;
        }
#pragma unroll
        for (int i = 0; i < kArVecPerThread; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v >= nvec) continue;
            if (c.mc_gather != nullptr) {
                // In-switch reduction: one load returns the sum of this vector over every rank (fp32
                // accumulation, bf16 result; the order of the additions is the switch's), one store per
                // 16 bytes delivers the sum and the call number to every rank.
                const uint8_t* src = c.mc_buf[parity] + (base + v) * 16;
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                             : "=r"(y[i][0]), "=r"(y[i][1]), "=r"(y[i][2]), "=r"(y[i][3]) : "l"(src) : "memory");
                uint8_t* dst = c.mc_gather + (base + v) * 32;
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst),
                             "f"(__uint_as_float(y[i][0])), "f"(__uint_as_float(call)), "f"(__uint_as_float(y[i][1])),
                             "f"(__uint_as_float(call))
                             : "memory");
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst + 16),
                             "f"(__uint_as_float(y[i][2])), "f"(__uint_as_float(call)), "f"(__uint_as_float(y[i][3])),
                             "f"(__uint_as_float(call))
                             : "memory");
                continue;
            }
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < c.world; ++r) {  // rank order
                const uint4 a = __ldcv(reinterpret_cast<const uint4*>(c.peer_buf[parity][r]) + base + v);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[2 * j] += bf16_lo(aw[j]);
                    acc[2 * j + 1] += bf16_hi(aw[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) y[i][j] = pack_bf16(acc[2 * j], acc[2 * j + 1]);
            // two bf16 pairs + call number per 16-byte store, to every peer
            const uint4 w0 = make_uint4(y[i][0], call, y[i][1], call);
            const uint4 w1 = make_uint4(y[i][2], call, y[i][3], call);
            for (int r = 0; r < c.world; ++r) {
                if (r == c.rank) continue;
                uint4* dst = reinterpret_cast<uint4*>(c.peer_gather[r]) + (base + v) * 2;
                asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(w0.x), "r"(w0.y),
                             "r"(w0.z), "r"(w0.w)
                             : "memory");
                asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + 1), "r"(w1.x), "r"(w1.y),
                             "r"(w1.z), "r"(w1.w)
                             : "memory");
            }
        }
    } else {
        const uint64_t t0 = global_timer_ns();
#pragma unroll
        for (int i = 0; i < kArVecPerThread; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v >= nvec) continue;
            const uint4* src = reinterpret_cast<const uint4*>(c.peer_gather[c.rank]) + (base + v) * 2;
            uint32_t spins = 0;
            for (;;) {
                uint4 w0, w1;
                asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "l"(src) : "memory");
                asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "l"(src + 1) : "memory");
                if (w0.y == call && w0.w == call && w1.y == call && w1.w == call) {
                    y[i][0] = w0.x; y[i][1] = w0.z; y[i][2] = w1.x; y[i][3] = w1.z;
                    break;
                }
                if ((++spins & 0xffu) == 0 && global_timer_ns() - t0 > c.wait_limit_ns) {
                    atomicExch(&status[kStatusTimeout], 403);
                    s_ok = 0;
                    y[i][0] = y[i][1] = y[i][2] = y[i][3] = 0u;
                    break;
                }
            }
        }
    }
    if (threadIdx.x == 0) c.self_counter[row] = call;
    __syncthreads();
    if (!s_ok) return;  // the reduced row never arrived: leave `residual` and `out` as they are

    // every rank: the same add + norm on the same sum
    float vals[kArVecPerThread][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kArVecPerThread; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v >= nvec) continue;
        if (MODE == 0) {
            reinterpret_cast<uint4*>(out)[base + v] = make_uint4(y[i][0], y[i][1], y[i][2], y[i][3]);
        } else {
            const uint4 rr = reinterpret_cast<const uint4*>(residual)[base + v];
            const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = bf16_lo(y[i][j]) + bf16_lo(rw[j]);
                const float hi = bf16_hi(y[i][j]) + bf16_hi(rw[j]);
                packed[j] = pack_bf16(lo, hi);
                vals[i][2 * j] = ROUND_FIRST ? bf16_lo(packed[j]) : lo;
                vals[i][2 * j + 1] = ROUND_FIRST ? bf16_hi(packed[j]) : hi;
            }
            reinterpret_cast<uint4*>(residual)[base + v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
    }
    if (MODE == 0) return;
    ss = warp_sum(ss);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    tot = warp_sum(tot);
    const float scale = rsqrtf(tot / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int i = 0; i < kArVecPerThread; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v >= nvec) continue;
        const uint4 w4 = reinterpret_cast<const uint4*>(weight)[v];
        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = pack_bf16(vals[i][2 * j] * scale * bf16_lo(ww[j]), vals[i][2 * j + 1] * scale * bf16_hi(ww[j]));
        reinterpret_cast<uint4*>(out)[base + v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

// Host object: this rank's exchange buffers and flag table, and the peers' mappings.
struct b200_comm {
    int rank = 0, world = 1, device = 0;
    int64_t buffer_bytes = 0;
    void* local_base = nullptr;       // [flags | counters | buffer 0 | buffer 1]
    void* peer_base[kMaxRanks] = {};  // mapped bases (own entry = local_base)
    bool connected = false;
    CommDevice dev = {};
    int64_t flags_bytes = 0, counters_bytes = 0;
    int two_shot_min_world = 8;   // B200_AR_TWO_SHOT_MIN_WORLD: groups of at least this size use the two-shot kernel
    uint64_t wait_limit_ns = 2000000000ull;  // 2 s, as every other bounded wait of the library
    bool loopback = false;        // every "peer" is this rank's own memory (time-out tests on one GPU)
    bool owns_memory = true;      // local_base came from cudaMalloc here (false: the caller's symmetric allocation)
    bool mapped_ipc = false;      // peer bases were opened from CUDA IPC handles
};

namespace {
int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }
}  // namespace

extern "C" {

int b200_comm_create(int rank, int world, int64_t buffer_bytes, b200_comm** out) {
    B200_CHECK_ARG(out, "comm_create: out is NULL");
    B200_CHECK_ARG(world >= 1 && world <= kMaxRanks, "comm_create: world size must be in [1, 8]");
    B200_CHECK_ARG(rank >= 0 && rank < world, "comm_create: rank out of range");
    B200_CHECK_ARG(buffer_bytes > 0, "comm_create: buffer_bytes must be positive");
    b200_comm* c = new b200_comm();
    c->rank = rank;
    c->world = world;
    B200_CHECK_CUDA(cudaGetDevice(&c->device));
    c->buffer_bytes = align_up(buffer_bytes, 256);
    c->flags_bytes = align_up(static_cast<int64_t>(kMaxCommBlocks) * kMaxRanks * 4, 256);
    c->counters_bytes = align_up(static_cast<int64_t>(kMaxCommBlocks) * 4, 256);
    if (const char* v = getenv("B200_AR_TWO_SHOT_MIN_WORLD")) c->two_shot_min_world = atoi(v);
    // [flags | counters | buffer 0 | buffer 1 | gather buffer (2 x: half of every word is the call number)]
    const int64_t total = c->flags_bytes + c->counters_bytes + 4 * c->buffer_bytes;
    if (cudaMalloc(&c->local_base, static_cast<size_t>(total)) != cudaSuccess ||
        cudaMemset(c->local_base, 0, static_cast<size_t>(total)) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) {
        set_last_error("comm_create: allocating %lld bytes failed: %s", static_cast<long long>(total),
                       cudaGetErrorString(cudaGetLastError()));
        delete c;
        return B200_ERR_CUDA;
    }
    c->peer_base[rank] = c->local_base;
    *out = c;
    return B200_OK;
}

int64_t b200_comm_region_bytes(int64_t buffer_bytes) {
    if (buffer_bytes <= 0) return -1;
    return align_up(static_cast<int64_t>(kMaxCommBlocks) * kMaxRanks * 4, 256) +
           align_up(static_cast<int64_t>(kMaxCommBlocks) * 4, 256) + 4 * align_up(buffer_bytes, 256);
}

int b200_comm_create_on(int rank, int world, int64_t buffer_bytes, void* region, b200_comm** out) {
    B200_CHECK_ARG(out && region, "comm_create_on: NULL argument");
    B200_CHECK_ARG(world >= 1 && world <= kMaxRanks, "comm_create_on: world size must be in [1, 8]");
    B200_CHECK_ARG(rank >= 0 && rank < world, "comm_create_on: rank out of range");
    B200_CHECK_ARG(buffer_bytes > 0, "comm_create_on: buffer_bytes must be positive");
    B200_CHECK_ARG((reinterpret_cast<uintptr_t>(region) & 255u) == 0, "comm_create_on: the region must be 256-byte aligned");
    b200_comm* c = new b200_comm();
    c->rank = rank;
    c->world = world;
    B200_CHECK_CUDA(cudaGetDevice(&c->device));
    c->buffer_bytes = align_up(buffer_bytes, 256);
    c->flags_bytes = align_up(static_cast<int64_t>(kMaxCommBlocks) * kMaxRanks * 4, 256);
    c->counters_bytes = align_up(static_cast<int64_t>(kMaxCommBlocks) * 4, 256);
    if (const char* v = getenv("B200_AR_TWO_SHOT_MIN_WORLD")) c->two_shot_min_world = atoi(v);
    c->local_base = region;
    c->owns_memory = false;
    c->peer_base[rank] = region;
    *out = c;
    return B200_OK;
}

static void comm_set_pointers(b200_comm* c, const void* multicast_base) {
    for (int r = 0; r < c->world; ++r) {
        char* base = static_cast<char*>(c->peer_base[r]);
        c->dev.peer_flags[r] = reinterpret_cast<uint32_t*>(base);
        for (int p = 0; p < 2; ++p)
            c->dev.peer_buf[p][r] = reinterpret_cast<const __nv_bfloat16*>(base + c->flags_bytes + c->counters_bytes +
                                                                          p * c->buffer_bytes);
        c->dev.peer_gather[r] = base + c->flags_bytes + c->counters_bytes + 2 * c->buffer_bytes;
    }
    const uint8_t* mc = static_cast<const uint8_t*>(multicast_base);
    for (int p = 0; p < 2; ++p)
        c->dev.mc_buf[p] = mc ? mc + c->flags_bytes + c->counters_bytes + p * c->buffer_bytes : nullptr;
    c->dev.mc_gather = mc ? const_cast<uint8_t*>(mc) + c->flags_bytes + c->counters_bytes + 2 * c->buffer_bytes : nullptr;
    c->dev.self_counter = reinterpret_cast<uint32_t*>(static_cast<char*>(c->local_base) + c->flags_bytes);
    c->dev.rank = c->rank;
    c->dev.world = c->world;
    c->dev.wait_limit_ns = c->wait_limit_ns;
    c->connected = true;
}

int b200_comm_connect_pointers(b200_comm* c, const void* const* peer_regions, const void* multicast_region) {
    B200_CHECK_ARG(c && peer_regions, "comm_connect_pointers: NULL argument");
    B200_CHECK_ARG(!c->connected, "comm_connect_pointers: already connected");
    for (int r = 0; r < c->world; ++r) {
        B200_CHECK_ARG(peer_regions[r] != nullptr, "comm_connect_pointers: rank %d has no region", r);
        if (r != c->rank) c->peer_base[r] = const_cast<void*>(peer_regions[r]);
    }
    comm_set_pointers(c, multicast_region);
    return B200_OK;
}

int b200_comm_uses_multicast(b200_comm* c) { return c && c->dev.mc_gather != nullptr ? 1 : 0; }

int b200_comm_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

int b200_comm_export(b200_comm* c, void* handle_out) {
    B200_CHECK_ARG(c && handle_out, "comm_export: NULL argument");
    cudaIpcMemHandle_t h;
    B200_CHECK_CUDA(cudaIpcGetMemHandle(&h, c->local_base));
    memcpy(handle_out, &h, sizeof(h));
    return B200_OK;
}

int b200_comm_connect(b200_comm* c, const void* all_handles) {
    B200_CHECK_ARG(c && all_handles, "comm_connect: NULL argument");
    B200_CHECK_ARG(!c->connected, "comm_connect: already connected");
    const char* hs = static_cast<const char*>(all_handles);
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, hs + static_cast<size_t>(r) * sizeof(h), sizeof(h));
        B200_CHECK_CUDA(cudaIpcOpenMemHandle(&c->peer_base[r], h, cudaIpcMemLazyEnablePeerAccess));
    }
    c->mapped_ipc = true;
    comm_set_pointers(c, nullptr);
    return B200_OK;
}

int b200_comm_set_wait_limit_ns(b200_comm* c, uint64_t ns) {
    B200_CHECK_ARG(c && ns > 0, "comm_set_wait_limit_ns: NULL communicator or zero limit");
    c->wait_limit_ns = ns;
    c->dev.wait_limit_ns = ns;
    return B200_OK;
}

int b200_comm_connect_loopback(b200_comm* c) {
    B200_CHECK_ARG(c, "comm_connect_loopback: NULL communicator");
    B200_CHECK_ARG(!c->connected, "comm_connect_loopback: already connected");
    for (int r = 0; r < c->world; ++r) c->peer_base[r] = c->local_base;
    c->loopback = true;
    comm_set_pointers(c, nullptr);
    return B200_OK;
}

int b200_comm_loopback_announce(b200_comm* c, uint32_t call_number, b200_stream_t stream) {
    B200_CHECK_ARG(c && c->connected && c->loopback, "comm_loopback_announce: not a loop-back communicator");
    // flag table [slots][kMaxRanks]: the word of source rank r in every slot
    std::vector<uint32_t> row(static_cast<size_t>(kMaxCommBlocks) * kMaxRanks);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200_CHECK_CUDA(cudaStreamSynchronize(s));
    B200_CHECK_CUDA(cudaMemcpy(row.data(), c->local_base, row.size() * 4, cudaMemcpyDeviceToHost));
    for (int slot = 0; slot < kMaxCommBlocks; ++slot)
        for (int r = 0; r < c->world; ++r)
            if (r != c->rank) row[static_cast<size_t>(slot) * kMaxRanks + r] = call_number;
    B200_CHECK_CUDA(cudaMemcpy(c->local_base, row.data(), row.size() * 4, cudaMemcpyHostToDevice));
    return B200_OK;
}

void* b200_comm_buffer(b200_comm* c, int parity) {
    if (!c || parity < 0 || parity > 1) return nullptr;
    return static_cast<char*>(c->local_base) + c->flags_bytes + c->counters_bytes + parity * c->buffer_bytes;
}

int b200_comm_destroy(b200_comm* c) {
    if (!c) return B200_OK;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->peer_base[r] && c->mapped_ipc) cudaIpcCloseMemHandle(c->peer_base[r]);
    if (c->local_base && c->owns_memory) cudaFree(c->local_base);
    delete c;
    return B200_OK;
}

}  // extern "C"

namespace b200 {

int launch_allreduce(b200_comm* c, int parity, int mode, void* out, void* residual, const void* weight,
                     int rows, int hidden, float eps, bool round_first, int* status, cudaStream_t stream) {
    if (!c || !c->connected) {
        set_last_error("all-reduce: the communicator is not connected");
        return B200_ERR_STATE;
    }
    if (hidden % 8 != 0 || hidden > 256 * 8 * kArVecPerThread) {
        set_last_error("all-reduce: row width %d must be a multiple of 8 and at most 8192", hidden);
        return B200_ERR_UNSUPPORTED;
    }
    if (static_cast<int64_t>(rows) * hidden * 2 > c->buffer_bytes) {
        set_last_error("all-reduce: %d x %d exceeds the exchange buffer", rows, hidden);
        return B200_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0) return B200_OK;
    if ((c->world >= c->two_shot_min_world || c->dev.mc_gather != nullptr) && rows <= kMaxCommBlocks) {
        auto k2 = mode == 0 ? allreduce_twoshot_kernel<0, false>
                            : (round_first ? allreduce_twoshot_kernel<1, true> : allreduce_twoshot_kernel<1, false>);
        B200_CHECK_CUDA(launch_kernel(k2, dim3(rows), dim3(256), 0, stream, dim3(1, 1, 1), c->dev, parity,
                                      static_cast<__nv_bfloat16*>(out), static_cast<__nv_bfloat16*>(residual),
                                      static_cast<const __nv_bfloat16*>(weight), rows, hidden, eps, status));
        return B200_OK;
    }
    // Every rank must launch the same number of CTAs: the handshake pairs CTA slots.
    const int grid = rows < kMaxCommBlocks ? rows : kMaxCommBlocks;
    auto kernel = mode == 0 ? allreduce_kernel<0, false>
                            : (round_first ? allreduce_kernel<1, true> : allreduce_kernel<1, false>);
    B200_CHECK_CUDA(launch_kernel(kernel, dim3(grid), dim3(256), 0, stream, dim3(1, 1, 1), c->dev, parity,
                                  static_cast<__nv_bfloat16*>(out), static_cast<__nv_bfloat16*>(residual),
                                  static_cast<const __nv_bfloat16*>(weight), rows, hidden, eps, status));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_allreduce(b200_comm* comm, int parity, void* out, int rows, int hidden, b200_stream_t stream) {
    B200_CHECK_ARG(comm && (rows == 0 || out), "allreduce: NULL argument");
    B200_CHECK_ARG(parity == 0 || parity == 1, "allreduce: parity must be 0 or 1");
    int err = B200_OK;
    int* status = device_status_words(&err);
    if (err != B200_OK) return err;
    return launch_allreduce(comm, parity, 0, out, nullptr, nullptr, rows, hidden, 0.f, false, status,
                            static_cast<cudaStream_t>(stream));
}

int b200_allreduce_fused_add_rmsnorm(b200_comm* comm, int parity, void* x_out, void* residual,
                                     const void* weight, int rows, int hidden, float eps,
                                     int round_sum_first, b200_stream_t stream) {
    B200_CHECK_ARG(comm && (rows == 0 || (x_out && residual && weight)), "allreduce_fused_add_rmsnorm: NULL argument");
    B200_CHECK_ARG(parity == 0 || parity == 1, "allreduce_fused_add_rmsnorm: parity must be 0 or 1");
    int err = B200_OK;
    int* status = device_status_words(&err);
    if (err != B200_OK) return err;
    return launch_allreduce(comm, parity, 1, x_out, residual, weight, rows, hidden, eps, round_sum_first != 0,
                            status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
