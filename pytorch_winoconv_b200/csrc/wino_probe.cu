// Calibration probe: how many clocks one tcgen05.mma (M = 128 per SM, K = 16, f16 operands, fp32 accumulate) costs
// as a function of the accumulator width N, the number of issuing threads, where the A operand lives (shared memory
// or tensor memory) and whether the instruction spans a CTA pair.  The planner's choices rest on these figures
// (an MMA with both operands in shared memory never takes fewer than ~40 clocks because of the 4 KB A-operand read,
// so accumulators narrower than 128 columns waste the pipe; with A in tensor memory N = 32 and 64 run at full rate),
// and the design notes quote them; this entry point lets anyone re-measure them on their own part.
// No counterpart in the reference.  Every wait is bounded; nothing is allocated.
#include <cuda_runtime.h>
#include <stdint.h>

#include "winoconv_b200.h"

namespace wino {
namespace probe {

__device__ long long g_probe_out[4];   // [0] makespan in clocks, [1] issue clocks of thread 0, [2] 1 if a wait gave up

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
constexpr uint32_t DESC_HI_SW64 = (uint32_t)(512 >> 4) | (1u << 14) | (4u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }

template <int CG>
__device__ __forceinline__ void mma_ss(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
  if (CG == 1)
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI_SW64), "r"(idesc), "r"(acc) : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI_SW64), "r"(idesc), "r"(acc) : "memory");
}
template <int CG>
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
  if (CG == 1)
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d), "r"(a_tmem), "r"(b_lo), "r"(DESC_HI_SW64), "r"(idesc), "r"(acc) : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d), "r"(a_tmem), "r"(b_lo), "r"(DESC_HI_SW64), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ uint32_t try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

constexpr int SMEM_BYTES = 132 * 1024;   // four 8 KB A slabs at 0, four 16 KB B slabs at 64 KB, 1 KB alignment slack

// Thread w (lane 0 of warp w, w < n_thr) issues n_mma MMAs into its own accumulator columns and commits; the result
// is the span from the first issue to the last completion.
template <int CG>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int n_mma, int N, int n_thr, int a_tmem) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t bars[4];
  __shared__ uint32_t tmem_slot;
  __shared__ long long t_start[4], t_end[4];
  __shared__ int gave_up;
  const uint32_t base = (smem_u32(smem) + 1023u) & ~1023u;
  for (int i = threadIdx.x; i < (SMEM_BYTES - 1024) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank = 0;
  if (CG == 2) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[i])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    gave_up = 0;
  }
  __syncthreads();
  if (CG == 2) cluster_sync_all();
  if (warp == 0) {
    if (CG == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CG == 2) cluster_sync_all();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  const uint32_t M = CG == 2 ? 256u : 128u;
  const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((M >> 4) << 24);
  // accumulator columns of thread w start at w * acc_stride; with A in tensor memory the last 32 columns hold A
  const int acc_stride = a_tmem ? (480 / n_thr) / 16 * 16 : 512 / n_thr;
  if (rank == 0 && lane == 0 && warp < n_thr) {
    const uint32_t a_lo = desc_lo(base + warp * 8192);
    const uint32_t b_lo = desc_lo(base + 65536 + warp * 16384);
    const uint32_t d = tmem + (uint32_t)(warp * acc_stride);
    const uint32_t a_t = tmem + 480u;
    const long long t0 = clock64();
    if (a_tmem) {
      for (int i = 0; i < n_mma; ++i) mma_ts<CG>(d, a_t + (uint32_t)((i & 3) * 8), b_lo + (uint32_t)((i & 1) * 2), idesc, i > 0 ? 1u : 0u);
    } else {
      for (int i = 0; i < n_mma; ++i) mma_ss<CG>(d, a_lo + (uint32_t)((i & 1) * 2), b_lo + (uint32_t)((i & 1) * 2), idesc, i > 0 ? 1u : 0u);
    }
    const long long t1 = clock64();
    if (CG == 1) {
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars[warp])) : "memory");
    } else {
      const uint16_t mask = 1;
      asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(&bars[warp])), "h"(mask) : "memory");
    }
    int spins = 0;
    while (!try_wait(smem_u32(&bars[warp]), 0u) && spins < (1 << 22)) ++spins;
    if (spins >= (1 << 22)) gave_up = 1;
    t_start[warp] = t0;
    t_end[warp] = clock64();
    if (warp == 0) g_probe_out[1] = t1 - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CG == 2) cluster_sync_all();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    long long s = t_start[0], e = t_end[0];
    for (int w = 1; w < n_thr; ++w) { s = min(s, t_start[w]); e = max(e, t_end[w]); }
    g_probe_out[0] = e - s;
    g_probe_out[2] = gave_up;
  }
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (CG == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

}  // namespace probe
}  // namespace wino

extern "C" int winoconv_probe_mma_rate(int cta_pair, int a_in_tmem, int n_cols, int n_threads, int n_mma,
                                       float *clocks_per_mma, float *issue_clocks_per_mma, void *stream) {
  using namespace wino::probe;
  if (!clocks_per_mma) return WINOCONV_ERR_INVALID_ARGUMENT;
  if (n_cols < 16 || n_cols > 256 || n_cols % 16 != 0 || (n_threads != 1 && n_threads != 2 && n_threads != 4) || n_mma < 1 || n_mma > 65536)
    return WINOCONV_ERR_INVALID_ARGUMENT;
  const int acc_stride = a_in_tmem ? (480 / n_threads) / 16 * 16 : 512 / n_threads;
  if (n_cols > acc_stride) return WINOCONV_ERR_UNSUPPORTED;     // the threads' accumulators would not fit tensor memory
  int st = winoconv_device_check();
  if (st != WINOCONV_OK) return st;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (cta_pair) {
    auto kern = mma_rate_kernel<2>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return WINOCONV_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1); cfg.blockDim = dim3(128, 1, 1); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, n_mma, n_cols, n_threads, a_in_tmem);
  } else {
    auto kern = mma_rate_kernel<1>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return WINOCONV_ERR_CUDA;
    kern<<<1, 128, SMEM_BYTES, s>>>(n_mma, n_cols, n_threads, a_in_tmem);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return WINOCONV_ERR_CUDA;
  long long out[4] = {0, 0, 0, 0};
  e = cudaMemcpyFromSymbolAsync(out, g_probe_out, sizeof(out), 0, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return WINOCONV_ERR_CUDA;
  if (out[2] != 0) return WINOCONV_ERR_TIMEOUT;
  *clocks_per_mma = (float)((double)out[0] / ((double)n_mma * n_threads));
  if (issue_clocks_per_mma) *issue_clocks_per_mma = (float)((double)out[1] / n_mma);
  return WINOCONV_OK;
}
