// Shared device/host helpers for the sm_100a token-loop kernels.
//
// Everything here is header-only so that each .cu file is a self-contained
// translation unit (no relocatable device code is needed to build the library).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_token_loop.h"

namespace b200 {

// ---------------------------------------------------------------------------
// Host-side helpers
// ---------------------------------------------------------------------------

// Status word array that kernels with bounded waits report into.  One small
// allocation per device, made on first use; see status.cu.
int* device_status_words(int* err);

// Number of SMs of the current device (cached).
int sm_count();

// Thread-local text of the last error a C-ABI call returned.
void set_last_error(const char* fmt, ...);

#define B200_CHECK_ARG(cond, ...)                    \
    do {                                             \
        if (!(cond)) {                               \
            ::b200::set_last_error(__VA_ARGS__);     \
            return B200_ERR_INVALID_ARGUMENT;        \
        }                                            \
    } while (0)

#define B200_CHECK_CUDA(expr)                                                        \
    do {                                                                             \
        cudaError_t e__ = (expr);                                                    \
        if (e__ != cudaSuccess) {                                                    \
            ::b200::set_last_error("%s failed: %s", #expr, cudaGetErrorString(e__)); \
            return B200_ERR_CUDA;                                                    \
        }                                                                            \
    } while (0)

#define B200_CHECK_LAUNCH() B200_CHECK_CUDA(cudaGetLastError())

// Whether kernels are launched as programmatic dependent launches (the step runner
// turns this on for its kernel chain: every kernel there executes griddepcontrol.wait
// before touching data a predecessor produces).  Per thread; off by default.
bool pdl_launches_enabled();
void set_pdl_launches(bool on);

// Kernels launched through launch_kernel by this thread so far (the step runner reports the
// difference across a step).
uint64_t kernel_launch_count();
void note_kernel_launch();

// One launch path for every kernel: cudaLaunchKernelEx, with the programmatic
// stream serialization attribute when enabled (and an optional cluster shape).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, dim3 cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned n = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = cluster.x;
        attrs[n].val.clusterDim.y = cluster.y;
        attrs[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    if (pdl_launches_enabled()) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    note_kernel_launch();
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int div_ceil(int a, int b) { return (a + b - 1) / b; }
static inline int64_t div_ceil64(int64_t a, int64_t b) { return (a + b - 1) / b; }

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// Device-side helpers
// ---------------------------------------------------------------------------

// Indices into the device status word array.
enum StatusWord : int {
    kStatusTimeout = 0,   // a bounded wait ran out (value: id of the wait site)
    kStatusBadIndex = 1,  // an index check failed (value: the offending index + 1)
};

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

__device__ __forceinline__ float round_bf16(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier --------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Longest time any single wait inside a kernel may take before the kernel gives
// up, records the wait site in the status word and unwinds.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

// Waits for the phase with the given parity to complete.  Returns false when the
// time limit ran out; the caller must then stop issuing work and unwind.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status,
                                                  int site) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xffu) == 0) {
            if (global_timer_ns() - t0 > kWaitLimitNs) {
                if (status) atomicExch(&status[kStatusTimeout], site);
                return false;
            }
        }
    }
    return true;
}

// ---- TMA (tiled tensor copies, never multicast) -----------------------------

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// c0 is the innermost (contiguous) coordinate; c0 * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int c0, int c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, int c0, int c1, int c2,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

// The same copy with an L2 eviction policy (from l2_policy_evict_first) for data read once.
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const void* tmap, int c0, int c1, int c2,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// ---- warp-level matrix helpers ----------------------------------------------

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                            uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte address of 16-byte chunk `chunk` (0..7) of a 128-byte row that starts at
// shared address `row_addr`, under the 128-byte TMA swizzle (the chunk index is
// XOR-ed with bits [7,10) of the row's shared address).
__device__ __forceinline__ uint32_t swz128(uint32_t row_addr, int chunk) {
    return row_addr + ((static_cast<uint32_t>(chunk) ^ ((row_addr >> 7) & 7u)) << 4);
}

// ---- programmatic dependent launch -------------------------------------------

// Blocks until every kernel this launch depends on has finished and flushed.
// A no-op when the kernel was launched without the programmatic attribute.
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the dependent launch start its prologue.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace b200
