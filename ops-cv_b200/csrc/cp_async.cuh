// cp.async helpers for per-thread asynchronous row queues: a thread copies its own piece of the next rows into a
// private shared-memory queue (one commit group per row) and consumes them in order with cp.async.wait_group.
#pragma once
#include <cstdint>

namespace opscv {

__device__ __forceinline__ void CpAsync16(void* smem, const void* gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(smem))),
                 "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void CpAsync4(void* smem, const void* gmem)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(smem))),
                 "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void CpAsyncWait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

} // namespace opscv
