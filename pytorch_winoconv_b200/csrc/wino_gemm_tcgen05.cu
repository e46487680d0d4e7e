// Per-position batched GEMM on the 5th-generation tensor cores (sm_100a):
//
//     m[p][t][k] = sum_c v[p][t][c] * u[p][k][c]        fp16 / bf16 in, fp32 accumulate
//
// Persistent: one CTA per SM walks 128 (tiles) x BN (output channels) blocks of the positions with a fixed stride.
//   warp 0      TMA producer: cp.async.bulk.tensor.3d loads of the V slab [128 x 64] and the U slab
//               [BN x 64] (both reduction-major, 128-byte swizzle) into a ring of shared-memory stages that runs on
//               across blocks, completion on an mbarrier per stage.  No cluster, no multicast.
//   warp 1      owns TMEM (tcgen05.alloc / dealloc) and issues tcgen05.mma.cta_group::1.kind::f16 (or kind::tf32)
//               from one thread: four MMAs per 128-byte slab, accumulator 128 lanes x BN fp32 columns, two of
//               them in TMEM; tcgen05.commit hands each stage back to the producer and each finished accumulator
//               to the epilogue.
//   warps 2..9  epilogue: tcgen05.ld of their 32-lane quarter (two warps per quarter, alternate chunks), 32 columns at a time, transposed through
//               shared memory so that each store instruction writes whole 128-byte rows of M; the accumulator
//               goes back to warp 1 as soon as its last columns are in registers.
//   warps 10..13 (three-tf32-product kind only) split every landed stage into hi / lo parts in shared memory.
// Ragged edges need no special code on the load side: TMA zero-fills rows beyond `tiles` / `k_out` and
// channels beyond `c_pad`; the epilogue masks its stores.
//
// Every mbarrier wait is bounded (about a second of SM clocks).  A wait that gives up records a code in
// g_device_error, raises the CTA's abort word so the other roles stop too, and the CTA still frees its
// TMEM and returns.
//
// Stands in for forwardAssign + cublasHgemmBatched (src/base_conv_launchers_half.cu:218-236; the
// reference accumulates in fp16 there) and cublasSgemmBatched (src/base_conv_launchers.cu:349-367).
#include <cuda.h>

#include <map>
#include <mutex>

#include "wino_common.cuh"
#include "wino_launch.h"

namespace wino {

// Error word of the bounded waits (0 = none).  Lives in this translation unit with its only writers.
__device__ unsigned int g_device_error = 0;

namespace tc {

constexpr int BM = 128;      // rows (tiles) per CTA == TMEM lanes
constexpr int BK = 64;       // reduction slab: 64 x 2 B = one 128-byte swizzle row
constexpr long long WAIT_LIMIT_CLOCKS = 2000000000LL;  // ~1 s at 1.9 GHz

enum ErrCode : unsigned { ERR_PRODUCER_EMPTY = 0x101, ERR_MMA_FULL = 0x102, ERR_EPI_ACC = 0x103, ERR_DRAIN = 0x104 };

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the CTA is aborting or the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile unsigned *abort_word, unsigned code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_word != 0u) return false;
    if (clock64() - start > WAIT_LIMIT_CLOCKS) {
      *abort_word = code;
      atomicCAS(&g_device_error, 0u, code);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Shared-memory matrix descriptor: reduction-major operand, 128-byte swizzle, rows 128 B apart, groups of
// eight rows 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <typename TM> struct StoreRow;
// 8 lanes x float4 cover the 32 columns of one row; 4 rows per instruction.
template <> struct StoreRow<float> {
  static constexpr int ROWS_PER_ITER = 4;
  static __device__ __forceinline__ void run(const float *stage, int lane, int iter, float *m_rows, long long ld,
                                             int rows_valid, int cols_valid) {
    const int r = iter * 4 + (lane >> 3), c = (lane & 7) * 4;
    if (r < rows_valid && c < cols_valid) {
      const float4 val = *reinterpret_cast<const float4 *>(stage + r * 36 + c);
      *reinterpret_cast<float4 *>(m_rows + r * ld + c) = val;
    }
  }
};
// 4 lanes x 8 values (16 bytes of 16-bit output) cover one row; 8 rows per instruction.
template <typename H> struct StoreRow16 {
  static constexpr int ROWS_PER_ITER = 8;
  static __device__ __forceinline__ void run(const float *stage, int lane, int iter, H *m_rows, long long ld,
                                             int rows_valid, int cols_valid) {
    const int r = iter * 8 + (lane >> 2), c = (lane & 3) * 8;
    if (r < rows_valid && c < cols_valid) {
      const float4 a = *reinterpret_cast<const float4 *>(stage + r * 36 + c);
      const float4 b = *reinterpret_cast<const float4 *>(stage + r * 36 + c + 4);
      float v[4] = {a.x, a.y, a.z, a.w}, w[4] = {b.x, b.y, b.z, b.w};
      VecIO<H, 4>::store(m_rows + r * ld + c, v);
      VecIO<H, 4>::store(m_rows + r * ld + c + 4, w);
    }
  }
};
template <> struct StoreRow<__half> : StoreRow16<__half> {};
template <> struct StoreRow<__nv_bfloat16> : StoreRow16<__nv_bfloat16> {};

// What the operands are and how a product is formed.
enum Kind : int { KIND_F16 = 0, KIND_TF32 = 1, KIND_TF32X3 = 2 };

// fp32 operands on the tensor cores: kind::tf32, plain or as three products of a hi / lo split.
// A tf32 multiply keeps 10 mantissa bits of each operand, which is not enough for the 1e-3 bound of the fp32 path
// (measured: see the cfg1 parity test).  Writing every operand as hi + lo, with hi the value rounded to tf32 and
// lo = x - hi (exact in fp32), the three products hi*hi + lo*hi + hi*lo leave an error of order 2^-21.  The split
// is made in shared memory: four warps rewrite each stage in place as it lands (hi over the loaded values, lo into a
// second copy at the same offsets, so the 128-byte swizzle carries over) and then hand it to the MMA thread.  V, U
// and the transforms that produce them are untouched: no second pass over HBM.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

constexpr int EPI_WARPS = 8;                                  // two per tensor-memory lane quarter: alternate 32-column chunks
constexpr int EPI_STAGING_BYTES = EPI_WARPS * 32 * 36 * 4;   // per epilogue warp 32 rows x (32 + 4 pad) floats

template <int BN, int KIND> struct PCfg {
  static constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128;      // rows of one 128-byte swizzle atom: 64 halves or 32 floats
  static constexpr int HALF_BYTES = A_BYTES + B_BYTES;              // what TMA loads per stage
  static constexpr int STAGE_BYTES = (KIND == KIND_TF32X3 ? 2 : 1) * HALF_BYTES;   // [A hi | B hi | A lo | B lo]
  static constexpr int FIXED_BYTES = EPI_STAGING_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/;
  static constexpr int MAX_STAGES = 8;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS + (KIND == KIND_TF32X3 ? 128 : 0);
  // CTAs that may share an SM: each holds 2 x BN of the 512 tensor-memory columns
  static constexpr int TMEM_CTAS = 512 / (2 * BN);
  static constexpr int smem_bytes(int stages) { return stages * STAGE_BYTES + FIXED_BYTES; }
  // stages of a CTA that shares its SM with ctas - 1 others
  static constexpr int stages_for(int ctas) {
    int st = (227 * 1024 / ctas - FIXED_BYTES) / STAGE_BYTES;
    return st > MAX_STAGES ? MAX_STAGES : st;
  }
};

// Persistent: a few CTAs per SM walk the (position, row block, column block) work tiles with a fixed stride.  The TMA
// ring runs on across tiles, and the accumulator is double-buffered in tensor memory (2 x BN columns), so the loads and
// MMAs of the next tile overlap the epilogue of this one and the set-up (tensor-memory allocation, barrier
// initialisation, descriptor fetch) is paid once per CTA instead of once per 128-row tile.  A short reduction runs
// with a short ring and several CTAs per SM (as many as the tensor-memory columns allow): its time is the epilogue's
// stores, and more epilogue warps per SM keep more of them in flight.
template <int BN, typename TM, int KIND>
__global__ void __launch_bounds__(PCfg<BN, KIND>::THREADS, 1)
    gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_u,
                           TM *__restrict__ m, int tiles, int c_pad, int k_out, int n_blocks, int m_blocks,
                           long long total_work, uint32_t idesc, int n_stages) {
  using C = PCfg<BN, KIND>;
  const int NS = n_stages;
  constexpr int BKE = KIND == KIND_F16 ? BK : 32;       // elements per 128-byte row of a stage
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;  // swizzled stages need 1024-byte alignment
  uint8_t *ring_ptr = smem_raw + (ring - raw);
  const int RING_BYTES = NS * C::STAGE_BYTES;
  float *staging = reinterpret_cast<float *>(ring_ptr + RING_BYTES);
  const uint32_t bars = ring + RING_BYTES + EPI_STAGING_BYTES;   // full[NS] empty[NS] split[NS] acc_full[2] acc_empty[2]
  volatile unsigned *abort_word = reinterpret_cast<volatile unsigned *>(ring_ptr + RING_BYTES + EPI_STAGING_BYTES + 384);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(ring_ptr + RING_BYTES + EPI_STAGING_BYTES + 388);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (NS + s); };
  auto split_bar = [&](int s) { return bars + 8u * (2 * NS + s); };
  auto acc_full = [&](int b) { return bars + 8u * (3 * NS + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (3 * NS + 2 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kb = (c_pad + BKE - 1) / BKE;
  const long long w0 = blockIdx.x, w_step = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(split_bar(s), 4);          // one arrival per splitting warp
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);           // the MMA thread's commit
      mbar_init(acc_empty(b), EPI_WARPS);  // one arrival per epilogue warp
    }
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // whole warp: two accumulators of BN fp32 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;
  const long long mn = (long long)m_blocks * n_blocks;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0, ph = 0;
      int s = 0;
      bool alive = true;
      for (long long w = w0; w < total_work && alive; w += w_step) {
        const int pos = (int)(w / mn);
        const int rem = (int)(w - (long long)pos * mn);
        const int m_blk = rem / n_blocks, n_blk = rem - m_blk * n_blocks;
        for (int kb = 0; kb < n_kb; ++kb, ++it, (++s == NS ? (s = 0, ph ^= 1u) : 0u)) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_word, ERR_PRODUCER_EMPTY)) { alive = false; break; }
          mbar_expect_tx(full_bar(s), (uint32_t)C::HALF_BYTES);
          const uint32_t a_dst = ring + s * C::STAGE_BYTES;
          tma_load_3d(a_dst, &map_v, full_bar(s), kb * BKE, m_blk * BM, pos);
          tma_load_3d(a_dst + C::A_BYTES, &map_u, full_bar(s), kb * BKE, n_blk * BN, pos);
        }
      }
      if (*abort_word != 0u) {
        // Aborting: nobody may be consuming any more.  Wait (bounded) until every load this thread issued
        // has landed, so no bulk copy is still writing shared memory when the CTA exits.
        for (uint32_t j = (it > (uint32_t)NS ? it - (uint32_t)NS : 0u); j < it; ++j) {
          const long long start = clock64();
          while (!mbar_try_wait(full_bar((int)(j % (uint32_t)NS)), (j / (uint32_t)NS) & 1u)) {
            if (clock64() - start > WAIT_LIMIT_CLOCKS) { atomicCAS(&g_device_error, 0u, (unsigned)ERR_DRAIN); break; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      uint32_t n_done = 0, ph = 0;
      int s = 0;
      bool alive = true;
      for (long long w = w0; w < total_work && alive; w += w_step, ++n_done) {
        const int buf = (int)(n_done & 1u);
        if (!mbar_wait(acc_empty(buf), ((n_done >> 1) & 1u) ^ 1u, abort_word, ERR_EPI_ACC)) { alive = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_acc + (uint32_t)(buf * BN);
        for (int kb = 0; kb < n_kb; ++kb, (++s == NS ? (s = 0, ph ^= 1u) : 0u)) {
          if (!mbar_wait(KIND == KIND_TF32X3 ? split_bar(s) : full_bar(s), ph, abort_word, ERR_MMA_FULL)) { alive = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_base = ring + s * C::STAGE_BYTES;
          const uint64_t a_hi = make_smem_desc(a_base), b_hi = make_smem_desc(a_base + C::A_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) {   // 16 halves or 8 floats along the reduction = 32 bytes = 2 descriptor address units
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            if (KIND == KIND_F16) {
              umma_f16(d, a_hi + 2u * k, b_hi + 2u * k, idesc, acc);
            } else if (KIND == KIND_TF32) {
              umma_tf32(d, a_hi + 2u * k, b_hi + 2u * k, idesc, acc);
            } else {
              const uint64_t a_lo = make_smem_desc(a_base + C::HALF_BYTES), b_lo = make_smem_desc(a_base + C::HALF_BYTES + C::A_BYTES);
              umma_tf32(d, a_lo + 2u * k, b_hi + 2u * k, idesc, acc);
              umma_tf32(d, a_hi + 2u * k, b_lo + 2u * k, idesc, 1u);
              umma_tf32(d, a_hi + 2u * k, b_hi + 2u * k, idesc, 1u);
            }
          }
          umma_commit(empty_bar(s));  // stage reusable once these MMAs have read it
        }
        umma_commit(acc_full(buf));   // accumulator complete (or whatever was issued, when aborting)
      }
    }
  } else if (warp >= 2 + EPI_WARPS) {
    // ---------------------------------------------------------------- hi / lo split (three-product kind only)
    const int st = threadIdx.x - (64 + 32 * EPI_WARPS);      // 0..127
    uint32_t ph = 0;
    int s = 0;
    bool alive = true;
    for (long long w = w0; w < total_work && alive; w += w_step) {
      for (int kb = 0; kb < n_kb; ++kb, (++s == NS ? (s = 0, ph ^= 1u) : 0u)) {
        unsigned got = 0;
        if (lane == 0) got = mbar_wait(full_bar(s), ph, abort_word, ERR_MMA_FULL) ? 1u : 0u;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (got == 0u) { alive = false; break; }
        float4 *hi = reinterpret_cast<float4 *>(ring_ptr + s * C::STAGE_BYTES);
        float4 *lo = reinterpret_cast<float4 *>(ring_ptr + s * C::STAGE_BYTES + C::HALF_BYTES);
#pragma unroll 4
        for (int i = st; i < C::HALF_BYTES / 16; i += 128) {
          const float4 x = hi[i];
          float4 h, l;
          h.x = tf32_round(x.x); h.y = tf32_round(x.y); h.z = tf32_round(x.z); h.w = tf32_round(x.w);
          l.x = x.x - h.x; l.y = x.y - h.y; l.z = x.z - h.z; l.w = x.w - h.w;
          hi[i] = h;
          lo[i] = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // these stores before the MMA's reads
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(split_bar(s)) : "memory");
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..9)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;   // which of the two warps of that quarter: even or odd 32-column chunks
    float *stage = staging + (warp - 2) * (32 * 36);
    const bool vec_ok = (k_out % 8) == 0;
    uint32_t n_done = 0;
    bool alive = true;
    for (long long w = w0; w < total_work && alive; w += w_step, ++n_done) {
      const int pos = (int)(w / mn);
      const int rem = (int)(w - (long long)pos * mn);
      const int m_blk = rem / n_blocks, n_blk = rem - m_blk * n_blocks;
      const int buf = (int)(n_done & 1u);
      unsigned got = 0;
      if (lane == 0) got = mbar_wait(acc_full(buf), (n_done >> 1) & 1u, abort_word, ERR_EPI_ACC) ? 1u : 0u;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got == 0u || *abort_word != 0u) { alive = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const long long row0 = (long long)m_blk * BM + q * 32;
      const int rows_valid = (int)max(0LL, min(32LL, (long long)tiles - row0));
      TM *m_rows = m + ((long long)pos * tiles + row0) * k_out + (long long)n_blk * BN;
      const int cols_here = min(BN, k_out - n_blk * BN);            // >= 1
      const int n_chunks = (cols_here + 31) / 32;
      if (half >= n_chunks) {            // nothing to read for this warp: its share of the hand-back
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
      }
      for (int ch = half; ch < n_chunks; ch += 2) {
        const int c0 = ch * 32;
        const int cols_valid = min(32, cols_here - c0);
        uint32_t r[32];
        tmem_ld_32x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c0), r);
        if (ch + 2 >= n_chunks) {        // this warp's last columns are in registers: hand the accumulator back to the MMA thread
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4 *>(stage + lane * 36 + 4 * j) =
              make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                          __uint_as_float(r[4 * j + 3]));
        __syncwarp();
        if (vec_ok) {
#pragma unroll
          for (int itr = 0; itr < 32 / StoreRow<TM>::ROWS_PER_ITER; ++itr)
            StoreRow<TM>::run(stage, lane, itr, m_rows + c0, (long long)k_out, rows_valid, cols_valid);
        } else {  // k_out not a multiple of 8: rows of M are not 16-byte aligned, store element-wise
          for (int rr = 0; rr < rows_valid; ++rr)
            if (lane < cols_valid) Elem<TM>::store(m_rows + (long long)rr * k_out + c0 + lane, stage[rr * 36 + lane]);
        }
        __syncwarp();
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)(2 * BN)) : "memory");
  }
}

// ---- F(4x4,3x3) input transform with the raw patches staged through shared memory by TMA ---------------------------
// V[pos][tile][c] = (B^T d B)[pos] for 16-bit layers whose channel count is a multiple of eight.  A persistent CTA walks
// blocks of 4 x 8 tiles x 64 channels: one warp loads the block's 18 x 34-pixel patch with one 4-D
// cp.async.bulk.tensor per block (out-of-bounds zero fill = the layer's padding) into a two-deep ring, twelve warps
// transform it -- a warp takes one tile at a time, its lanes the 32 channel pairs of the block, so the shared-memory
// reads are conflict-free and every store is a whole 128-byte line of V -- on packed fp32 pairs.  The global loads, whose
// latency bound the one-thread-per-tile kernel, are the TMA engine's; the warps only compute and store.
constexpr int XT_TH = 4, XT_TW = 8;                              // tiles per block
constexpr int XT_PH = 4 * XT_TH + 2, XT_PW = 4 * XT_TW + 2;     // pixels per patch: 18 x 34
constexpr int XT_C = 64;                                         // channels per patch: 128 bytes per pixel
constexpr int XT_PATCH_BYTES = XT_PH * XT_PW * XT_C * 2;
constexpr int XT_BUFS = 2;
constexpr int XT_SMEM_BYTES = XT_BUFS * XT_PATCH_BYTES + 1024 + 256;
constexpr int XT_WARPS = 12;                                     // transforming warps
constexpr int XT_THREADS = 32 + 32 * XT_WARPS;

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

struct XtGeom {
  int N, C, Cp, nH, nW, pH, pW;
  int n_rb, n_cb, n_chb;      // blocks of tile rows, tile columns and channels
  long long T, n_items;
};

template <typename T>
__global__ void __launch_bounds__(XT_THREADS, 1) input_f43_tma_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                       T *__restrict__ v, const __grid_constant__ XtGeom g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  const uint8_t *base_ptr = smem_raw + (base - raw);
  const uint32_t bars = base + XT_BUFS * XT_PATCH_BYTES;   // full[2] empty[2]
  volatile unsigned *abort_word = reinterpret_cast<volatile unsigned *>(const_cast<uint8_t *>(base_ptr) + XT_BUFS * XT_PATCH_BYTES + 64);
  auto full_bar = [&](int b) { return bars + 8u * b; };
  auto empty_bar = [&](int b) { return bars + 8u * (XT_BUFS + b); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int b = 0; b < XT_BUFS; ++b) {
      mbar_init(full_bar(b), 1);
      mbar_init(empty_bar(b), XT_WARPS);   // one arrival per transforming warp
    }
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const long long per_img = (long long)g.n_rb * g.n_cb * g.n_chb;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (long long w = blockIdx.x; w < g.n_items; w += gridDim.x, ++it) {
        const int b = (int)(it & 1u);
        if (!mbar_wait(empty_bar(b), ((it >> 1) & 1u) ^ 1u, abort_word, ERR_PRODUCER_EMPTY)) break;
        const int n = (int)(w / per_img);
        int rem = (int)(w - (long long)n * per_img);
        const int chb = rem % g.n_chb; rem /= g.n_chb;
        const int cb = rem % g.n_cb, rb = rem / g.n_cb;
        mbar_expect_tx(full_bar(b), (uint32_t)XT_PATCH_BYTES);
        tma_load_4d(base + b * XT_PATCH_BYTES, &map_x, full_bar(b), chb * XT_C, cb * (4 * XT_TW) - g.pW, rb * (4 * XT_TH) - g.pH, n);
      }
      if (*abort_word != 0u) {   // let the loads still in flight land before the shared memory goes away
        for (uint32_t j = (it > 2u ? it - 2u : 0u); j < it; ++j) {
          const long long start = clock64();
          while (!mbar_try_wait(full_bar((int)(j & 1u)), (j >> 1) & 1u)) {
            if (clock64() - start > WAIT_LIMIT_CLOCKS) { atomicCAS(&g_device_error, 0u, (unsigned)ERR_DRAIN); break; }
          }
        }
      }
    }
  } else {
    const int wi = warp - 1;               // 0..XT_WARPS-1: the block's tiles are dealt to the warps in turn
    const long long v_pos_stride = g.T * g.Cp;
    uint32_t it = 0;
    bool alive = true;
    for (long long w = blockIdx.x; w < g.n_items && alive; w += gridDim.x, ++it) {
      const int b = (int)(it & 1u);
      unsigned got = 0;
      if (lane == 0) got = mbar_wait(full_bar(b), (it >> 1) & 1u, abort_word, ERR_MMA_FULL) ? 1u : 0u;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got == 0u) { alive = false; break; }
      const int n = (int)(w / per_img);
      int rem = (int)(w - (long long)n * per_img);
      const int chb = rem % g.n_chb; rem /= g.n_chb;
      const int cb = rem % g.n_cb, rb = rem / g.n_cb;
      const int c = chb * XT_C + 2 * lane;             // this lane's channel pair
      const uint8_t *patch = base_ptr + b * XT_PATCH_BYTES + lane * 4;
      const int vh = min(XT_TH, g.nH - rb * XT_TH), vw = min(XT_TW, g.nW - cb * XT_TW);   // tiles of the block inside the image
      if (c < g.Cp) {
#pragma unroll 1
        for (int t = wi; t < vh * vw; t += XT_WARPS) {
          const int tr = t / vw, tw_warp = t - tr * vw;
          const int th = rb * XT_TH + tr, tw = cb * XT_TW + tw_warp;
          uint64_t q[36];
#pragma unroll
          for (int r = 0; r < 6; ++r)
#pragma unroll
            for (int sx = 0; sx < 6; ++sx) {
              const uint32_t raw2 = *reinterpret_cast<const uint32_t *>(patch + ((4 * tr + r) * XT_PW + 4 * tw_warp + sx) * (XT_C * 2));
              float f[2];
              VecIO<T, 2>::load(reinterpret_cast<const T *>(&raw2), f);
              q[r * 6 + sx] = f2_pack(f[0], f[1]);
            }
#pragma unroll
          for (int r = 0; r < 6; ++r) Xf<4, 3>::template bt2<1>(&q[r * 6]);
#pragma unroll
          for (int sx = 0; sx < 6; ++sx) Xf<4, 3>::template bt2<6>(&q[sx]);
          T *dst = v + (((long long)n * g.nH + th) * g.nW + tw) * g.Cp + c;
#pragma unroll
          for (int i = 0; i < 36; ++i) {
            float o[2];
            f2_unpack(q[i], o[0], o[1]);
            VecIO<T, 2>::store(dst, o);
            dst += v_pos_stride;
          }
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(b)) : "memory");
    }
  }
}

// ---- F(4x4,3x3) output transform with the products staged through shared memory by TMA -----------------------------
// y = A^T M A (+ bias, ReLU) for 16-bit layers whose output channel count is a multiple of eight.  The same scheme as
// the input side: a persistent CTA walks blocks of 8 tiles x 64 channels; one warp loads the block's 36 positions with
// one 3-D cp.async.bulk.tensor ([64 channels, 8 tiles, 36 positions] of M) into a two-deep ring, eight warps take one
// tile each -- lanes = the 32 channel pairs -- transform on packed fp32 pairs and store whole 128-byte runs of y.
constexpr int YT_TILES = 8;
constexpr int YT_C = 64;
constexpr int YT_WARPS = 8;
constexpr int YT_THREADS = 32 + 32 * YT_WARPS;
template <typename TM> struct YtCfg {
  static constexpr int BOX_BYTES = 36 * YT_TILES * YT_C * (int)sizeof(TM);
  static constexpr int SMEM_BYTES = 2 * BOX_BYTES + 1024 + 256;
};

struct YtGeom {
  int K, nH, nW, oH, oW;
  int n_chb;
  unsigned epilogue;
  long long T, n_items;
};

template <typename TM> struct LoadPair;
template <> struct LoadPair<float> {
  static __device__ __forceinline__ uint64_t get(const uint8_t *p) { return *reinterpret_cast<const uint64_t *>(p); }
};
template <> struct LoadPair<__half> {
  static __device__ __forceinline__ uint64_t get(const uint8_t *p) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(p));
    return f2_pack(f.x, f.y);
  }
};
template <> struct LoadPair<__nv_bfloat16> {
  static __device__ __forceinline__ uint64_t get(const uint8_t *p) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
    return f2_pack(f.x, f.y);
  }
};

template <typename T, typename TM>
__global__ void __launch_bounds__(YT_THREADS, 1) output_f43_tma_kernel(const __grid_constant__ CUtensorMap map_m,
                                                                        T *__restrict__ y, const T *__restrict__ bias,
                                                                        const __grid_constant__ YtGeom g) {
  using C = YtCfg<TM>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  const uint8_t *base_ptr = smem_raw + (base - raw);
  const uint32_t bars = base + 2 * C::BOX_BYTES;   // full[2] empty[2]
  volatile unsigned *abort_word = reinterpret_cast<volatile unsigned *>(const_cast<uint8_t *>(base_ptr) + 2 * C::BOX_BYTES + 64);
  auto full_bar = [&](int b) { return bars + 8u * b; };
  auto empty_bar = [&](int b) { return bars + 8u * (2 + b); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(full_bar(b), 1);
      mbar_init(empty_bar(b), YT_WARPS);
    }
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (long long w = blockIdx.x; w < g.n_items; w += gridDim.x, ++it) {
        const int b = (int)(it & 1u);
        if (!mbar_wait(empty_bar(b), ((it >> 1) & 1u) ^ 1u, abort_word, ERR_PRODUCER_EMPTY)) break;
        const long long tg = w / g.n_chb;
        const int chb = (int)(w - tg * g.n_chb);
        mbar_expect_tx(full_bar(b), (uint32_t)C::BOX_BYTES);
        tma_load_3d(base + b * C::BOX_BYTES, &map_m, full_bar(b), chb * YT_C, (int)(tg * YT_TILES), 0);
      }
      if (*abort_word != 0u) {   // let the loads still in flight land before the shared memory goes away
        for (uint32_t j = (it > 2u ? it - 2u : 0u); j < it; ++j) {
          const long long start = clock64();
          while (!mbar_try_wait(full_bar((int)(j & 1u)), (j >> 1) & 1u)) {
            if (clock64() - start > WAIT_LIMIT_CLOCKS) { atomicCAS(&g_device_error, 0u, (unsigned)ERR_DRAIN); break; }
          }
        }
      }
    }
  } else {
    const int tl = warp - 1;               // this warp's tile of the block
    const bool relu = (g.epilogue & WINOCONV_EPI_RELU) != 0;
    const bool has_bias = (g.epilogue & WINOCONV_EPI_BIAS) != 0;
    uint32_t it = 0;
    bool alive = true;
    for (long long w = blockIdx.x; w < g.n_items && alive; w += gridDim.x, ++it) {
      const int b = (int)(it & 1u);
      unsigned got = 0;
      if (lane == 0) got = mbar_wait(full_bar(b), (it >> 1) & 1u, abort_word, ERR_MMA_FULL) ? 1u : 0u;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got == 0u) { alive = false; break; }
      const long long tg = w / g.n_chb;
      const int chb = (int)(w - tg * g.n_chb);
      const long long tile = tg * YT_TILES + tl;
      const int k = chb * YT_C + 2 * lane;
      if (tile < g.T && k < g.K) {
        const uint8_t *src = base_ptr + b * C::BOX_BYTES + (tl * YT_C + 2 * lane) * (int)sizeof(TM);
        uint64_t q[36], t1[24], o[16];
#pragma unroll
        for (int p = 0; p < 36; ++p) q[p] = LoadPair<TM>::get(src + p * (YT_TILES * YT_C * (int)sizeof(TM)));
#pragma unroll
        for (int r = 0; r < 6; ++r) Xf<4, 3>::template at2<1, 1>(&q[r * 6], &t1[r * 4]);      // along W: 6 -> 4 per row
#pragma unroll
        for (int cidx = 0; cidx < 4; ++cidx) Xf<4, 3>::template at2<4, 4>(&t1[cidx], &o[cidx]);   // along H
        uint64_t bv = f2_pack(0.f, 0.f);
        if (has_bias) {
          float bf[2];
          VecIO<T, 2>::load(bias + k, bf);
          bv = f2_pack(bf[0], bf[1]);
        }
        const unsigned t32 = (unsigned)tile;
        const unsigned tw = t32 % (unsigned)g.nW, r2 = t32 / (unsigned)g.nW;
        const unsigned th = r2 % (unsigned)g.nH, n = r2 / (unsigned)g.nH;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const int oh = (int)th * 4 + a;
          if (oh < g.oH) {
            T *rowp = y + (((long long)n * g.oH + oh) * g.oW + (long long)tw * 4) * g.K + k;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              if ((int)tw * 4 + cc < g.oW) {
                float f[2];
                f2_unpack(f2_add(o[a * 4 + cc], bv), f[0], f[1]);
                if (relu) { f[0] = fmaxf(f[0], 0.f); f[1] = fmaxf(f[1], 0.f); }
                VecIO<T, 2>::store(rowp + (long long)cc * g.K, f);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(b)) : "memory");
    }
  }
}

// ---- host side --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rows x c_pad operand per position, reduction innermost: dims {c_pad, rows, positions}.
static bool make_operand_map(CUtensorMap *map, int dtype, const void *base, int c_pad, long long rows, int positions,
                             int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  const cuuint64_t esz = dtype == WINOCONV_F32 ? 4ull : 2ull;
  const cuuint64_t dims[3] = {(cuuint64_t)c_pad, (cuuint64_t)rows, (cuuint64_t)positions};
  const cuuint64_t strides[2] = {(cuuint64_t)c_pad * esz, (cuuint64_t)c_pad * esz * (cuuint64_t)rows};
  const cuuint32_t box[3] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows, 1u};   // one 128-byte swizzle row
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUtensorMapDataType dt = dtype == WINOCONV_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == WINOCONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return enc(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int device_sm_count() {
  static std::mutex mu;
  static std::map<int, int> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(mu);
  auto f = cache.find(dev);
  if (f != cache.end()) return f->second;
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 0;
  cache[dev] = n;
  return n;
}

template <int BN, typename TM, int KIND>
static cudaError_t run(int dtype, int positions, long long tiles, int c_pad, int k_out, const void *v, const void *u,
                       void *m, cudaStream_t s, const char **detail) {
  using C = PCfg<BN, KIND>;
  CUtensorMap map_v, map_u;
  if (!make_operand_map(&map_v, dtype, v, c_pad, tiles, positions, BM) ||
      !make_operand_map(&map_u, dtype, u, c_pad, k_out, positions, BN)) {
    *detail = "cuTensorMapEncodeTiled failed (operands must be 16-byte aligned, c_pad a multiple of 8)";
    return cudaErrorInvalidValue;
  }
  auto kern = gemm_persistent_kernel<BN, TM, KIND>;
  // CTAs per SM: one with a deep ring for a long reduction; two with short rings for a reduction of one or two slabs,
  // whose time is the stores of M.  WINOCONV_GEMM_CTAS overrides (experiments; at most what the tensor memory allows).
  const int n_kb = (c_pad + (KIND == KIND_F16 ? 64 : 32) - 1) / (KIND == KIND_F16 ? 64 : 32);
  static const int ctas_env = [] { const char *v = getenv("WINOCONV_GEMM_CTAS"); return v && *v ? atoi(v) : 0; }();
  int ctas = (n_kb <= 2 && C::TMEM_CTAS >= 2) ? 2 : 1;   // measured: a reduction of four slabs already wants the deep ring
  if (ctas_env >= 1) ctas = ctas_env < C::TMEM_CTAS ? ctas_env : C::TMEM_CTAS;
  while (ctas > 1 && C::stages_for(ctas) < 2) --ctas;
  int n_stages = C::stages_for(ctas);
  // a ring no deeper than two tiles' worth of slabs, but deep enough that no more CTAs fit an SM than planned
  while (n_stages > 2 && n_stages > 2 * n_kb && C::smem_bytes(n_stages - 1) > 227 * 1024 / (ctas + 1)) --n_stages;
  const int smem_bytes = C::smem_bytes(n_stages);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_bytes(C::stages_for(1)));
  if (e != cudaSuccess) { *detail = "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed"; return e; }
  const int n_blocks = (k_out + BN - 1) / BN;
  const long long m_blocks = (tiles + BM - 1) / BM;
  if (m_blocks * n_blocks > 0x7fffffffLL) { *detail = "too many tile blocks for one launch"; return cudaErrorInvalidConfiguration; }
  const long long total = m_blocks * n_blocks * positions;
  const int sms = device_sm_count();
  if (sms <= 0) { *detail = "no device"; return cudaErrorNoDevice; }
  // instruction descriptor: D = f32, A = B = f16 (0) / bf16 (1) / tf32 (2), both reduction-major, N >> 3, M >> 4
  const uint32_t fmt = KIND != KIND_F16 ? 2u : (dtype == WINOCONV_F16 ? 0u : 1u);
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  const long long slots = (long long)sms * ctas;
  const unsigned grid = (unsigned)(total < slots ? total : slots);
  kern<<<grid, C::THREADS, smem_bytes, s>>>(map_v, map_u, (TM *)m, (int)tiles, c_pad, k_out, n_blocks, (int)m_blocks, total, idesc, n_stages);
  return cudaGetLastError();
}

// Wider than 128 output channels: 256-wide blocks read V once per 256 channels, 128-wide blocks fill the last round of
// the SMs better on a small problem; take whichever needs less time in whole rounds (a 256-wide block counts double).
static bool prefer_bn128(int positions, long long tiles, int k_out) {
  const int sms = device_sm_count();
  if (sms <= 0) return false;
  const long long m_blocks = (tiles + BM - 1) / BM;
  const long long w256 = m_blocks * positions * ((k_out + 255) / 256), w128 = m_blocks * positions * ((k_out + 127) / 128);
  return (w128 + sms - 1) / sms < 2 * ((w256 + sms - 1) / sms);
}

template <typename TM>
static cudaError_t pick_bn(int dtype, int positions, long long tiles, int c_pad, int k_out, const void *v,
                           const void *u, void *m, cudaStream_t s, const char **detail) {
  if (k_out <= 64) return run<64, TM, KIND_F16>(dtype, positions, tiles, c_pad, k_out, v, u, m, s, detail);
  if (k_out <= 128 || prefer_bn128(positions, tiles, k_out))
    return run<128, TM, KIND_F16>(dtype, positions, tiles, c_pad, k_out, v, u, m, s, detail);
  return run<256, TM, KIND_F16>(dtype, positions, tiles, c_pad, k_out, v, u, m, s, detail);
}

template <typename T>
static cudaError_t run_input_f43_tma(const Geom &g, int dtype, const void *x, void *v, cudaStream_t s, const char **detail) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { *detail = "cuTensorMapEncodeTiled unavailable"; return cudaErrorNotSupported; }
  CUtensorMap map_x;
  const cuuint64_t dims[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N};
  const cuuint64_t st[3] = {(cuuint64_t)g.C * 2ull, (cuuint64_t)g.C * 2ull * g.W, (cuuint64_t)g.C * 2ull * g.W * g.H};
  const cuuint32_t box[4] = {(cuuint32_t)XT_C, (cuuint32_t)XT_PW, (cuuint32_t)XT_PH, 1u};
  const cuuint32_t es[4] = {1u, 1u, 1u, 1u};
  const CUtensorMapDataType dt = dtype == WINOCONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (enc(&map_x, dt, 4, const_cast<void *>(x), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    *detail = "cuTensorMapEncodeTiled failed for the input of the F(4x4,3x3) transform";
    return cudaErrorInvalidValue;
  }
  XtGeom q;
  q.N = g.N; q.C = g.C; q.Cp = g.Cp; q.nH = g.nH; q.nW = g.nW; q.pH = g.pH; q.pW = g.pW;
  q.n_rb = (g.nH + XT_TH - 1) / XT_TH; q.n_cb = (g.nW + XT_TW - 1) / XT_TW; q.n_chb = (g.Cp + XT_C - 1) / XT_C;
  q.T = g.T; q.n_items = (long long)g.N * q.n_rb * q.n_cb * q.n_chb;
  auto kern = input_f43_tma_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, XT_SMEM_BYTES);
  if (e != cudaSuccess) { *detail = "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed"; return e; }
  const int sms = device_sm_count();
  if (sms <= 0) { *detail = "no device"; return cudaErrorNoDevice; }
  const unsigned grid = (unsigned)(q.n_items < sms ? q.n_items : sms);
  kern<<<grid, XT_THREADS, XT_SMEM_BYTES, s>>>(map_x, (T *)v, q);
  return cudaGetLastError();
}

template <typename T, typename TM>
static cudaError_t run_output_f43_tma(const Geom &g, int product_dtype, const void *m, void *y, const void *bias,
                                      cudaStream_t s, const char **detail) {
  using C = YtCfg<TM>;
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { *detail = "cuTensorMapEncodeTiled unavailable"; return cudaErrorNotSupported; }
  CUtensorMap map_m;
  const cuuint64_t esz = sizeof(TM);
  const cuuint64_t dims[3] = {(cuuint64_t)g.K, (cuuint64_t)g.T, 36ull};
  const cuuint64_t st[2] = {(cuuint64_t)g.K * esz, (cuuint64_t)g.K * esz * (cuuint64_t)g.T};
  const cuuint32_t box[3] = {(cuuint32_t)YT_C, (cuuint32_t)YT_TILES, 36u};
  const cuuint32_t es[3] = {1u, 1u, 1u};
  const CUtensorMapDataType dt = product_dtype == WINOCONV_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : product_dtype == WINOCONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (enc(&map_m, dt, 3, const_cast<void *>(m), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    *detail = "cuTensorMapEncodeTiled failed for the products of the F(4x4,3x3) output transform";
    return cudaErrorInvalidValue;
  }
  YtGeom q;
  q.K = g.K; q.nH = g.nH; q.nW = g.nW; q.oH = g.oH; q.oW = g.oW; q.epilogue = g.epilogue; q.T = g.T;
  q.n_chb = (g.K + YT_C - 1) / YT_C;
  q.n_items = ((g.T + YT_TILES - 1) / YT_TILES) * q.n_chb;
  auto kern = output_f43_tma_kernel<T, TM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) { *detail = "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed"; return e; }
  const int sms = device_sm_count();
  if (sms <= 0) { *detail = "no device"; return cudaErrorNoDevice; }
  const unsigned grid = (unsigned)(q.n_items < sms ? q.n_items : sms);
  kern<<<grid, YT_THREADS, C::SMEM_BYTES, s>>>(map_m, (T *)y, (const T *)bias, q);
  return cudaGetLastError();
}

}  // namespace tc

bool output_f43_tma_applies(const Geom &g, int dtype, int product_dtype, const void *m, long long t0, long long n_tiles) {
  return (dtype == WINOCONV_F16 || dtype == WINOCONV_BF16) && (product_dtype == WINOCONV_F32 || product_dtype == dtype) &&
         g.mD == 1 && g.mH == 4 && g.mW == 4 && g.n_pieces == 1 && g.oD == 1 && g.K % 8 == 0 &&
         (g.epilogue & WINOCONV_EPI_POOL2) == 0 && t0 == 0 && n_tiles == g.T && g.T < (1LL << 31) &&
         (reinterpret_cast<uintptr_t>(m) & 15u) == 0;
}

cudaError_t launch_output_f43_tma(const Geom &g, int dtype, int product_dtype, const void *m, void *y, const void *bias,
                                  cudaStream_t s, const char **detail) {
  *detail = "";
  if (dtype == WINOCONV_F16) {
    if (product_dtype == WINOCONV_F32) return tc::run_output_f43_tma<__half, float>(g, product_dtype, m, y, bias, s, detail);
    return tc::run_output_f43_tma<__half, __half>(g, product_dtype, m, y, bias, s, detail);
  }
  if (product_dtype == WINOCONV_F32) return tc::run_output_f43_tma<__nv_bfloat16, float>(g, product_dtype, m, y, bias, s, detail);
  return tc::run_output_f43_tma<__nv_bfloat16, __nv_bfloat16>(g, product_dtype, m, y, bias, s, detail);
}

bool input_f43_tma_applies(const Geom &g, int dtype, const void *x, long long t0, long long n_tiles) {
  return (dtype == WINOCONV_F16 || dtype == WINOCONV_BF16) && g.mD == 1 && g.mH == 4 && g.mW == 4 && g.n_pieces == 1 &&
         g.D == 1 && g.C % 8 == 0 && g.C == g.Cp && t0 == 0 && n_tiles == g.T && g.T < (1LL << 31) &&
         (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
}

cudaError_t launch_input_f43_tma(const Geom &g, int dtype, const void *x, void *v, cudaStream_t s, const char **detail) {
  *detail = "";
  if (dtype == WINOCONV_F16) return tc::run_input_f43_tma<__half>(g, dtype, x, v, s, detail);
  return tc::run_input_f43_tma<__nv_bfloat16>(g, dtype, x, v, s, detail);
}


cudaError_t launch_gemm_tf32(int split, int positions, long long tiles, int c_pad, int k_out, const void *v,
                             const void *u, void *m, cudaStream_t s, const char **detail) {
  *detail = "";
  if (positions <= 0 || tiles <= 0) return cudaSuccess;
  if (c_pad % 8 != 0 || positions > 65535 || tiles > 0x7fffffffLL) { *detail = "c_pad must be a multiple of 8; positions <= 65535"; return cudaErrorInvalidValue; }
  if (split) {   // the split stages are twice as large: 128 output channels per CTA at most
    if (k_out <= 64) return tc::run<64, float, tc::KIND_TF32X3>(WINOCONV_F32, positions, tiles, c_pad, k_out, v, u, m, s, detail);
    return tc::run<128, float, tc::KIND_TF32X3>(WINOCONV_F32, positions, tiles, c_pad, k_out, v, u, m, s, detail);
  }
  if (k_out <= 64) return tc::run<64, float, tc::KIND_TF32>(WINOCONV_F32, positions, tiles, c_pad, k_out, v, u, m, s, detail);
  if (k_out <= 128 || tc::prefer_bn128(positions, tiles, k_out))
    return tc::run<128, float, tc::KIND_TF32>(WINOCONV_F32, positions, tiles, c_pad, k_out, v, u, m, s, detail);
  return tc::run<256, float, tc::KIND_TF32>(WINOCONV_F32, positions, tiles, c_pad, k_out, v, u, m, s, detail);
}

cudaError_t read_and_clear_device_error(cudaStream_t s, unsigned int *code) {
  unsigned int host = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&host, g_device_error, sizeof(host), 0, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemcpyToSymbolAsync(g_device_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  *code = host;
  return e;
}

cudaError_t launch_gemm_tcgen05(int dtype, int product_dtype, int positions, long long tiles, int c_pad, int k_out,
                                const void *v, const void *u, void *m, cudaStream_t s, const char **detail) {
  *detail = "";
  if (positions <= 0 || tiles <= 0) return cudaSuccess;
  if (dtype != WINOCONV_F16 && dtype != WINOCONV_BF16) { *detail = "tcgen05 GEMM takes f16 or bf16 operands"; return cudaErrorInvalidValue; }
  if (c_pad % 8 != 0 || positions > 65535 || tiles > 0x7fffffffLL) { *detail = "c_pad must be a multiple of 8; positions <= 65535"; return cudaErrorInvalidValue; }
  if (product_dtype == WINOCONV_F32) return tc::pick_bn<float>(dtype, positions, tiles, c_pad, k_out, v, u, m, s, detail);
  if (dtype == WINOCONV_F16) return tc::pick_bn<__half>(dtype, positions, tiles, c_pad, k_out, v, u, m, s, detail);
  return tc::pick_bn<__nv_bfloat16>(dtype, positions, tiles, c_pad, k_out, v, u, m, s, detail);
}

}  // namespace wino
