// Shared device helpers of the sm_100a kernels.
//
// Every launcher in this library is an extern "C" function that takes raw device
// pointers, sizes and a cudaStream_t, launches on that stream, and returns the
// cudaError_t of the launch as an int (0 = success, negative = an argument the
// kernel refuses).  Nothing here allocates or synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PB_EXPORT extern "C" __attribute__((visibility("default")))

// Refusals (returned instead of a wrong result).
#define PB_ERR_BAD_DTYPE (-2)
#define PB_ERR_BAD_SIZE (-3)
#define PB_ERR_TOO_LARGE (-4)

enum PbDtype { PB_F32 = 0, PB_BF16 = 1 };

namespace pb {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads, in a fixed order (lane tree, then warp 0's
// lane tree over the warp partials), so the result does not depend on scheduling.
// `scratch` needs 32 floats.  Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();   // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

inline int launch_status() { return (int)cudaPeekAtLastError(); }

// Bounds checks of the debug build (-DPB_CHECK_BOUNDS; PULSAR_CHECK_BOUNDS=1 when the library is built): every page
// id and slot that a kernel takes from a block table or a slot array is checked against the pool's size before it
// becomes an address.  A bad one is recorded in the caller's error word (the largest code seen: 2 = a page id in a
// block table, 3 = a slot) and the access is skipped: a read takes page 0 instead, a write is dropped.  The host sets
// what the next launches check against (pb_set_pool_bounds); without the flag the checks compile to nothing.
// (The reference checks its arguments on the host, pulsar-core/src/kernels/paged_common.cu:172-272, and has one device
// assertion, pulsar-core/inc/pulsar/kernels/attn_params.cuh:130.)
struct PoolBounds {
    int n_pages;             // pages of the pool the next launches read and write; <= 0: unchecked
    unsigned int* error;     // device word; null: unchecked
};
PoolBounds pool_bounds_now();            // host side: what pb_set_pool_bounds set last (zeros in a build without the flag)

__device__ __forceinline__ bool page_ok(int page, const PoolBounds& b) {
#ifdef PB_CHECK_BOUNDS
    if (b.error != nullptr && b.n_pages > 0 && (page < 0 || page >= b.n_pages)) {
        atomicMax(b.error, 2u);
        return false;
    }
#endif
    return true;
}
__device__ __forceinline__ bool slot_ok(int slot, int page_size, const PoolBounds& b) {
#ifdef PB_CHECK_BOUNDS
    if (b.error != nullptr && b.n_pages > 0 && slot >= b.n_pages * page_size) {        // negative: "no slot", skipped anyway
        atomicMax(b.error, 3u);
        return false;
    }
#endif
    return true;
}

// Programmatic dependent launch.  A kernel launched through launch_pdl may be brought onto the
// SMs while the kernel before it on the stream is finishing: as soon as every block of that
// kernel has called pdl_trigger (or exited).  It must call pdl_wait before it touches anything
// an earlier kernel writes (or reads and later overwrites); pdl_wait returns once the preceding
// kernel has completed and its writes are visible.  Every kernel of the chain waits first thing,
// so completion is transitive; kernels trigger late, after their main loop, so that the next
// kernel's launch overlaps only this kernel's tail.  Both calls do nothing in a kernel that was
// launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();      // PULSAR_PDL=0 launches every kernel the ordinary way

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace pb
