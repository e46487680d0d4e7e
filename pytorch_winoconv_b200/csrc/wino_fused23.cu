// Fused F(2x2, 3x3) Winograd / DWM forward for f16 / bf16 on sm_100a: one persistent kernel does the tile
// gather (zero padding, DWM piece offsets, stride-2 polyphase addressing), the input transform B^T d B, the
// per-position GEMMs on tcgen05 tensor cores with TMEM accumulators, the output transform A^T m A, the
// bias / ReLU / 2x2 max-pool epilogue and the store.  Neither the transformed input V nor the products M
// ever exist in global memory.
//
// DWM inside the GEMM.  Every piece is taken as a 3x3 sub-kernel (zero taps where the kernel ends), so all
// pieces share the same 16 Winograd positions and the same A^T; because A^T(.)A is linear, the sum over
// pieces moves in front of it:  Y = A^T ( sum_q sum_c U_q[c] * V_q[c] ) A.  Pieces (and, for 3-D, the depth
// taps, which are applied directly with a depth output block of 1) therefore become extra slabs of the GEMM
// reduction: the flattened reduction index is r = q * Cp + c.  The reference instead runs every piece as its
// own transform -> GEMM -> transform chain and adds the results in a separate kernel
// (src/base_conv_launchers.cu:338-381, src/split_kernel.cu:184-203).
//
// Work item = 128 tiles x 32 output channels; all 16 position accumulators (16 x 32 fp32 columns) fill the
// SM's 512 TMEM columns.  Per 64-wide reduction slab and per position row i_h one shared-memory stage holds
// the A operand of 4 positions (4 x [128 tiles x 64], 128-byte swizzle, written by the producer warps) and the
// B operand (4 x [32 channels x 64] of the transformed filter, TMA).
//   warps 0-7    producers: gather + transform, st.shared into the swizzled layout, fence.proxy.async, arrive
//   warp  8      TMEM alloc; one thread issues tcgen05.mma (M=128, N=32, K=16) and the commits
//   warp  9      one thread issues the TMA loads of the filter slabs
//   warps 10-13  epilogue: tcgen05.ld -> A^T m A -> bias / ReLU / pool -> shared-memory staging -> 64-byte row stores
// All mbarrier waits are bounded; a wait that gives up records a code in the device error word and the CTA
// still frees its TMEM and returns.
#include <cuda.h>

#include <algorithm>

#include "wino_common.cuh"
#include "wino_launch.h"

namespace wino {

// Error word of this translation unit's bounded waits (0 = none).
__device__ unsigned int g_fused_error = 0;

namespace fused {

__device__ __forceinline__ void record_device_error(unsigned code) { atomicCAS(&g_fused_error, 0u, code); }

constexpr int BM = 128, BN = 32, BK = 64, UMMA_K = 16;
constexpr int POS_PER_STAGE = 4;
constexpr int A_POS_BYTES = BM * BK * 2;            // 16 KB: one position's [128 x 64] slab
constexpr int B_POS_BYTES = BN * BK * 2;            //  4 KB
constexpr int STAGE_A_BYTES = POS_PER_STAGE * A_POS_BYTES;
constexpr int STAGE_B_BYTES = POS_PER_STAGE * B_POS_BYTES;
constexpr int STAGE_BYTES = STAGE_A_BYTES + STAGE_B_BYTES;   // 80 KB
constexpr int STAGES = 2;
constexpr int RING_BYTES = STAGES * STAGE_BYTES;             // 160 KB
constexpr int OUT_STAGE_BYTES = 4 * 32 * 4 * BN * 2;         // 4 warps x 32 tiles x 4 pixels x 32 ch x 2 B = 32 KB
constexpr int SMEM_BYTES = RING_BYTES + OUT_STAGE_BYTES + 1024 + 256;
constexpr int N_PRODUCER_THREADS = 256;
constexpr int N_THREADS = 448;
constexpr long long WAIT_LIMIT_CLOCKS = 2000000000LL;

enum ErrCode : unsigned { ERR_PROD_EMPTY = 0x201, ERR_TMA_EMPTY = 0x202, ERR_MMA_FULL = 0x203, ERR_MMA_ACC = 0x204, ERR_EPI_ACC = 0x205 };

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile unsigned *abort_word, unsigned code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_word != 0u) return false;
    if (clock64() - start > WAIT_LIMIT_CLOCKS) {
      *abort_word = code;
      record_device_error(code);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {  // reduction-major, SWIZZLE_128B, SBO 1024
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_x4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
}

// 8 packed 16-bit values (one 16-byte vector of channels)
template <typename T> struct Pack;
template <> struct Pack<__half> {
  using V2 = __half2;
  static __device__ __forceinline__ V2 add(V2 a, V2 b) { return __hadd2(a, b); }
  static __device__ __forceinline__ V2 sub(V2 a, V2 b) { return __hsub2(a, b); }
  static __device__ __forceinline__ V2 from_floats(float a, float b) { return __floats2half2_rn(a, b); }
};
template <> struct Pack<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  static __device__ __forceinline__ V2 add(V2 a, V2 b) { return __hadd2(a, b); }
  static __device__ __forceinline__ V2 sub(V2 a, V2 b) { return __hsub2(a, b); }
  static __device__ __forceinline__ V2 from_floats(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <typename T> struct __align__(16) Vec8 { typename Pack<T>::V2 h[4]; };

template <typename T> __device__ __forceinline__ Vec8<T> vec_zero() {
  Vec8<T> v;
  uint4 z = make_uint4(0u, 0u, 0u, 0u);
  *reinterpret_cast<uint4 *>(&v) = z;
  return v;
}
template <typename T> __device__ __forceinline__ Vec8<T> vec_add(const Vec8<T> &a, const Vec8<T> &b) {
  Vec8<T> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.h[i] = Pack<T>::add(a.h[i], b.h[i]);
  return r;
}
template <typename T> __device__ __forceinline__ Vec8<T> vec_sub(const Vec8<T> &a, const Vec8<T> &b) {
  Vec8<T> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.h[i] = Pack<T>::sub(a.h[i], b.h[i]);
  return r;
}

// 8 channels of one input pixel (zero outside the image / beyond C).  VEC: C is a multiple of 8 and x is
// 16-byte aligned, so the vector is one 16-byte load; otherwise channel by channel.
template <typename T, bool VEC>
__device__ __forceinline__ Vec8<T> load_px(const T *__restrict__ x, const FGeom &g, int n, int id, int ih, int iw, int c0) {
  if ((unsigned)id >= (unsigned)g.D || (unsigned)ih >= (unsigned)g.H || (unsigned)iw >= (unsigned)g.W) return vec_zero<T>();
  const T *p = x + ((((long long)n * g.D + id) * g.H + ih) * g.W + iw) * g.C + c0;
  Vec8<T> v;
  if (VEC) {
    *reinterpret_cast<uint4 *>(&v) = __ldg(reinterpret_cast<const uint4 *>(p));
  } else {
    T e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = (c0 + i < g.C) ? p[i] : T(0.f);
    *reinterpret_cast<uint4 *>(&v) = *reinterpret_cast<const uint4 *>(e);
  }
  return v;
}

struct TileRef { int n, od, ih0, iw0, th, tw; bool valid; };

__device__ __forceinline__ TileRef decode_tile(const FGeom &g, long long t) {
  TileRef r;
  r.valid = t < g.T;
  if (!r.valid) t = 0;
  r.tw = (int)(t % g.nW); t /= g.nW;
  r.th = (int)(t % g.nH); t /= g.nH;
  r.od = (int)(t % g.oD); t /= g.oD;
  r.n = (int)t;
  r.ih0 = g.sH * 2 * r.th - g.pH;
  r.iw0 = g.sW * 2 * r.tw - g.pW;
  return r;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(N_THREADS, 1) fused23_kernel(const __grid_constant__ CUtensorMap map_u,
                                                                const T *__restrict__ x, T *__restrict__ y,
                                                                const T *__restrict__ bias,
                                                                const __grid_constant__ FGeom g, int n_mblocks,
                                                                int n_nblocks, uint32_t idesc) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  uint8_t *ring_ptr = smem_raw + (ring - raw);
  uint8_t *out_stage = ring_ptr + RING_BYTES;
  const uint32_t bars = ring + RING_BYTES + OUT_STAGE_BYTES;   // full[2], empty[2], acc_full, acc_empty
  volatile unsigned *abort_word = reinterpret_cast<volatile unsigned *>(ring_ptr + RING_BYTES + OUT_STAGE_BYTES + 128);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(ring_ptr + RING_BYTES + OUT_STAGE_BYTES + 132);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * STAGES), acc_empty = bars + 8u * (2 * STAGES + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = n_mblocks * n_nblocks;
  const int n_chunks = (g.R + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), N_PRODUCER_THREADS + 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 128);
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  if (warp < 8) {
    // ------------------------------------------------------------------ producers
    const int v = threadIdx.x & 7;          // 16-byte vector (8 reduction indices) within the 64-wide slab
    const int r0 = threadIdx.x >> 3;        // rows r0, r0 + 32, r0 + 64, r0 + 96 of the tile block
    uint32_t it = 0;
    bool alive = true;
    for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
      const int m_blk = item / n_nblocks;
      TileRef tr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) tr[i] = decode_tile(g, (long long)m_blk * BM + r0 + 32 * i);
      for (int j = 0; j < n_chunks && alive; ++j) {
        const int flat = j * BK + v * 8;
        const int q = flat / g.Cp;
        const int c0 = flat - q * g.Cp;
        const bool active = q < g.P && c0 < g.C;
        int kd = 0, oh = 0, ow = 0;
        if (active) {
          const FPiece pc = g.pieces[q];
          kd = pc.kd;
          oh = g.sH * pc.st_h + pc.ph_h;     // row offset of the piece's window inside the tile's footprint
          ow = g.sW * pc.st_w + pc.ph_w;
        }
#pragma unroll 1
        for (int ih_pos = 0; ih_pos < 4 && alive; ++ih_pos) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, abort_word, ERR_PROD_EMPTY)) { alive = false; break; }
          // B^T row ih_pos of F(2,3): (0,-2) (1,+2) (2,-1) (1,-3)
          const int ra = (ih_pos == 0) ? 0 : ((ih_pos == 2) ? 2 : 1);
          const int rb = (ih_pos == 0) ? 2 : ((ih_pos == 1) ? 2 : ((ih_pos == 2) ? 1 : 3));
          const bool plus = ih_pos == 1;
          uint8_t *a_stage = ring_ptr + s * STAGE_BYTES;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = r0 + 32 * i;
            Vec8<T> d[4];
            if (active && tr[i].valid) {
              const int id = g.sD * tr[i].od + kd - g.pD;
              const int iha = tr[i].ih0 + oh + g.sH * ra, ihb = tr[i].ih0 + oh + g.sH * rb;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int iw = tr[i].iw0 + ow + g.sW * k;
                const Vec8<T> xa = load_px<T, VEC>(x, g, tr[i].n, id, iha, iw, c0);
                const Vec8<T> xb = load_px<T, VEC>(x, g, tr[i].n, id, ihb, iw, c0);
                d[k] = plus ? vec_add<T>(xa, xb) : vec_sub<T>(xa, xb);
              }
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) d[k] = vec_zero<T>();
            }
            // along W: v0 = d0 - d2, v1 = d1 + d2, v2 = d2 - d1, v3 = d1 - d3
            const Vec8<T> o0 = vec_sub<T>(d[0], d[2]), o1 = vec_add<T>(d[1], d[2]);
            const Vec8<T> o2 = vec_sub<T>(d[2], d[1]), o3 = vec_sub<T>(d[1], d[3]);
            // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
            const uint32_t off = (uint32_t)row * 128u + (uint32_t)((v ^ (row & 7)) << 4);
            *reinterpret_cast<uint4 *>(a_stage + 0 * A_POS_BYTES + off) = *reinterpret_cast<const uint4 *>(&o0);
            *reinterpret_cast<uint4 *>(a_stage + 1 * A_POS_BYTES + off) = *reinterpret_cast<const uint4 *>(&o1);
            *reinterpret_cast<uint4 *>(a_stage + 2 * A_POS_BYTES + off) = *reinterpret_cast<const uint4 *>(&o2);
            *reinterpret_cast<uint4 *>(a_stage + 3 * A_POS_BYTES + off) = *reinterpret_cast<const uint4 *>(&o3);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // make the generic-proxy stores visible to the MMA
          mbar_arrive(full_bar(s));
          ++it;
        }
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, n_done = 0;
      bool alive = true;
      for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x, ++n_done) {
        if (!mbar_wait(acc_empty, (n_done & 1u) ^ 1u, abort_word, ERR_MMA_ACC)) { alive = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int j = 0; j < n_chunks && alive; ++j) {
          for (int ih_pos = 0; ih_pos < 4; ++ih_pos) {
            const int s = it % STAGES;
            if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, abort_word, ERR_MMA_FULL)) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_base = ring + s * STAGE_BYTES, b_base = a_base + STAGE_A_BYTES;
#pragma unroll
            for (int k = 0; k < POS_PER_STAGE; ++k) {
              const uint64_t adesc = make_smem_desc(a_base + k * A_POS_BYTES);
              const uint64_t bdesc = make_smem_desc(b_base + k * B_POS_BYTES);
              const uint32_t d_col = tmem_acc + (uint32_t)((ih_pos * 4 + k) * BN);
#pragma unroll
              for (int kk = 0; kk < BK / UMMA_K; ++kk)
                umma_f16(d_col, adesc + 2u * kk, bdesc + 2u * kk, idesc, (j > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(s));
            ++it;
          }
        }
        umma_commit(acc_full);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ filter loads
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
        const int n_blk = item % n_nblocks;
        for (int j = 0; j < n_chunks && alive; ++j) {
          for (int ih_pos = 0; ih_pos < 4; ++ih_pos) {
            const int s = it % STAGES;
            if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1u) ^ 1u, abort_word, ERR_TMA_EMPTY)) { alive = false; break; }
            mbar_expect_tx(full_bar(s), (uint32_t)STAGE_B_BYTES);
            const uint32_t b_base = ring + s * STAGE_BYTES + STAGE_A_BYTES;
#pragma unroll
            for (int k = 0; k < POS_PER_STAGE; ++k)
              tma_load_3d(b_base + k * B_POS_BYTES, &map_u, full_bar(s), j * BK, n_blk * BN, ih_pos * 4 + k);
            ++it;
          }
        }
      }
      if (*abort_word != 0u) {   // let any load still in flight land before the CTA's shared memory goes away
        const long long start = clock64();
        while (clock64() - start < 2000000LL) { }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int qd = warp & 3;                     // TMEM lane quarter of this warp
    const int row = qd * 32 + lane;
    T *stage = reinterpret_cast<T *>(out_stage) + (size_t)(warp - 10) * (32 * 4 * BN);
    const bool relu = (g.epilogue & WINOCONV_EPI_RELU) != 0;
    const bool has_bias = (g.epilogue & WINOCONV_EPI_BIAS) != 0;
    const bool pool = (g.epilogue & WINOCONV_EPI_POOL2) != 0;
    const int n_px = pool ? 1 : 4;
    uint32_t n_done = 0;
    bool alive = true;
    for (int item = blockIdx.x; item < n_items && alive; item += gridDim.x, ++n_done) {
      const int m_blk = item / n_nblocks, n_blk = item % n_nblocks;
      unsigned got = 0;
      if (lane == 0) got = mbar_wait(acc_full, n_done & 1u, abort_word, ERR_EPI_ACC) ? 1u : 0u;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got == 0u) { alive = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t t_lane = tmem_acc + ((uint32_t)(qd * 32) << 16);
#pragma unroll 1
      for (int cb = 0; cb < BN / 4; ++cb) {
        uint32_t m[16][4];
#pragma unroll
        for (int p = 0; p < 16; ++p) tmem_ld_x4(t_lane + (uint32_t)(p * BN + cb * 4), m[p]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float o[4][4];   // [pixel a*2+b][channel]
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float t[4][2];   // after the W transform: rows i, columns b
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float m0 = __uint_as_float(m[i * 4 + 0][c]), m1 = __uint_as_float(m[i * 4 + 1][c]);
            const float m2 = __uint_as_float(m[i * 4 + 2][c]), m3 = __uint_as_float(m[i * 4 + 3][c]);
            t[i][0] = m0 + m1 + m2;
            t[i][1] = m1 - m2 - m3;
          }
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            o[0 * 2 + b][c] = t[0][b] + t[1][b] + t[2][b];
            o[1 * 2 + b][c] = t[1][b] - t[2][b] - t[3][b];
          }
        }
        const int kbase = n_blk * BN + cb * 4;
        float bv[4] = {0.f, 0.f, 0.f, 0.f};
        if (has_bias) {
#pragma unroll
          for (int c = 0; c < 4; ++c) if (kbase + c < g.K) bv[c] = Elem<T>::load(bias + kbase + c);
        }
        if (pool) {
          float r[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            r[c] = fmaxf(fmaxf(o[0][c], o[1][c]), fmaxf(o[2][c], o[3][c])) + bv[c];
            if (relu) r[c] = fmaxf(r[c], 0.f);
          }
          VecIO<T, 4>::store(stage + (size_t)lane * BN + cb * 4, r);
        } else {
#pragma unroll
          for (int px = 0; px < 4; ++px) {
            float r[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              r[c] = o[px][c] + bv[c];
              if (relu) r[c] = fmaxf(r[c], 0.f);
            }
            VecIO<T, 4>::store(stage + ((size_t)lane * 4 + px) * BN + cb * 4, r);
          }
        }
      }
      // accumulators are in registers / shared memory now: hand TMEM back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(acc_empty);
      __syncwarp();
      // staged [tile][pixel][32 ch] -> global: 4 lanes x 16 B cover one pixel's 64-byte channel run
      const int k0 = n_blk * BN;
      const int total_px = 32 * n_px;
      const bool vec_ok = (g.K % 8) == 0;
      for (int e = lane; e < total_px * 4; e += 32) {
        const int pix = e >> 2, part = e & 3;
        const int tl = pix / n_px, px = pix - tl * n_px;
        const long long tile = (long long)m_blk * BM + qd * 32 + tl;
        if (tile >= g.T) continue;
        const TileRef tr = decode_tile(g, tile);
        int yh, yw;
        if (pool) { yh = tr.th; yw = tr.tw; if (yh >= g.yH || yw >= g.yW) continue; }
        else { yh = 2 * tr.th + (px >> 1); yw = 2 * tr.tw + (px & 1); if (yh >= g.oH || yw >= g.oW) continue; }
        const int kk = k0 + part * 8;
        if (kk >= g.K) continue;
        const T *src = stage + (size_t)pix * BN + part * 8;
        T *dst = y + ((((long long)tr.n * g.oD + tr.od) * g.yH + yh) * g.yW + yw) * g.K + kk;
        if (vec_ok) {
          *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src);
        } else {
          for (int c = 0; c < 8 && kk + c < g.K; ++c) dst[c] = src[c];
        }
      }
      __syncwarp();
    }
    (void)row;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 8) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// Few input channels (C < 8, e.g. an RGB first layer): the reduction P * C is far shorter than one 64-wide
// MMA slab, so the same F(2x2,3x3)-window formulation runs as fp32 FMAs instead.  A 128-thread block keeps the
// whole transformed filter in shared memory (fp32, [16][P*C][K]), transforms the input windows of a few tiles
// into shared memory, then each thread accumulates the 16 positions of one tile for four output channels,
// applies A^T m A and the epilogue and stores.  x, y and the filter are the only global traffic.
// ---------------------------------------------------------------------------------------------------------
namespace smallc {
constexpr int THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(THREADS) fused23_smallc_kernel(const T *__restrict__ x, const T *__restrict__ u,
                                                                 T *__restrict__ y, const T *__restrict__ bias,
                                                                 const __grid_constant__ FGeom g, int reff, int kgroups,
                                                                 int tb, long long n_groups) {
  extern __shared__ float sm[];
  const int Kp = kgroups * 4;
  float *Us = sm;                          // [16][reff][Kp]
  float *Vs = sm + (size_t)16 * reff * Kp; // [tb][16][reff]
  const int tid = threadIdx.x;
  for (int idx = tid; idx < 16 * reff * Kp; idx += THREADS) {
    const int pos = idx / (reff * Kp), rem = idx - pos * (reff * Kp);
    const int r = rem / Kp, k = rem - r * Kp;
    const int q = r / g.C, c = r - q * g.C;
    Us[idx] = (k < g.K) ? Elem<T>::load(u + ((long long)pos * g.K + k) * g.R + q * g.Cp + c) : 0.f;
  }
  __syncthreads();
  const int tl = tid / kgroups, kg = tid - tl * kgroups;
  const bool relu = (g.epilogue & WINOCONV_EPI_RELU) != 0;
  const bool pool = (g.epilogue & WINOCONV_EPI_POOL2) != 0;
  for (long long grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
    // ---- input windows -> Vs
    for (int task = tid; task < tb * reff; task += THREADS) {
      const int t_local = task / reff, r = task - t_local * reff;
      const int q = r / g.C, c = r - q * g.C;
      const long long tile = grp * tb + t_local;
      float d[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) d[i] = 0.f;
      if (tile < g.T) {
        const TileRef tr = decode_tile(g, tile);
        const FPiece pc = g.pieces[q];
        const int id = g.sD * tr.od + pc.kd - g.pD;
        const int ihb = tr.ih0 + g.sH * pc.st_h + pc.ph_h, iwb = tr.iw0 + g.sW * pc.st_w + pc.ph_w;
        if ((unsigned)id < (unsigned)g.D) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int ih = ihb + g.sH * i;
            if ((unsigned)ih >= (unsigned)g.H) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int iw = iwb + g.sW * j;
              if ((unsigned)iw < (unsigned)g.W)
                d[i * 4 + j] = Elem<T>::load(x + ((((long long)tr.n * g.D + id) * g.H + ih) * g.W + iw) * g.C + c);
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) Xf<2, 3>::bt<1>(&d[i * 4]);
#pragma unroll
      for (int j = 0; j < 4; ++j) Xf<2, 3>::bt<4>(&d[j]);
      float *dst = Vs + (size_t)t_local * 16 * reff + r;
#pragma unroll
      for (int p = 0; p < 16; ++p) dst[p * reff] = d[p];
    }
    __syncthreads();
    // ---- 16 positions x 4 channels per thread
    const long long tile = grp * tb + tl;
    if (tl < tb && tile < g.T) {
      float acc[16][4];
#pragma unroll
      for (int p = 0; p < 16; ++p)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[p][c] = 0.f;
      const float *vs = Vs + (size_t)tl * 16 * reff;
      const float *us = Us + kg * 4;
#pragma unroll
      for (int p = 0; p < 16; ++p) {
        for (int r = 0; r < reff; ++r) {
          const float v = vs[p * reff + r];
          const float4 w4 = *reinterpret_cast<const float4 *>(us + ((size_t)p * reff + r) * Kp);
          acc[p][0] = fmaf(v, w4.x, acc[p][0]);
          acc[p][1] = fmaf(v, w4.y, acc[p][1]);
          acc[p][2] = fmaf(v, w4.z, acc[p][2]);
          acc[p][3] = fmaf(v, w4.w, acc[p][3]);
        }
      }
      const int k0 = kg * 4;
      float bv[4] = {0.f, 0.f, 0.f, 0.f};
      if (g.epilogue & WINOCONV_EPI_BIAS) {
#pragma unroll
        for (int c = 0; c < 4; ++c) if (k0 + c < g.K) bv[c] = Elem<T>::load(bias + k0 + c);
      }
      float o[4][4];   // [pixel a*2+b][channel]
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float t[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          t[i][0] = acc[i * 4 + 0][c] + acc[i * 4 + 1][c] + acc[i * 4 + 2][c];
          t[i][1] = acc[i * 4 + 1][c] - acc[i * 4 + 2][c] - acc[i * 4 + 3][c];
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          o[0 * 2 + b][c] = t[0][b] + t[1][b] + t[2][b];
          o[1 * 2 + b][c] = t[1][b] - t[2][b] - t[3][b];
        }
      }
      const TileRef tr = decode_tile(g, tile);
      const bool vec_ok = (g.K % 4) == 0;
      auto store_px = [&](int yh, int yw, const float (&r)[4]) {
        T *dst = y + ((((long long)tr.n * g.oD + tr.od) * g.yH + yh) * g.yW + yw) * g.K + k0;
        if (vec_ok) {
          VecIO<T, 4>::store(dst, r);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) if (k0 + c < g.K) Elem<T>::store(dst + c, r[c]);
        }
      };
      if (k0 < g.K) {
        if (pool) {
          if (tr.th < g.yH && tr.tw < g.yW) {
            float r[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              r[c] = fmaxf(fmaxf(o[0][c], o[1][c]), fmaxf(o[2][c], o[3][c])) + bv[c];
              if (relu) r[c] = fmaxf(r[c], 0.f);
            }
            store_px(tr.th, tr.tw, r);
          }
        } else {
#pragma unroll
          for (int px = 0; px < 4; ++px) {
            const int yh = 2 * tr.th + (px >> 1), yw = 2 * tr.tw + (px & 1);
            if (yh < g.oH && yw < g.oW) {
              float r[4];
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                r[c] = o[px][c] + bv[c];
                if (relu) r[c] = fmaxf(r[c], 0.f);
              }
              store_px(yh, yw, r);
            }
          }
        }
      }
    }
    __syncthreads();
  }
}

// shared memory of the small-C kernel, or 0 when the shape does not fit it
static size_t plan_smem(const FGeom &g, int *reff, int *kgroups, int *tb) {
  *reff = g.P * g.C;
  *kgroups = (g.K + 3) / 4;
  if (g.C >= 8 || *kgroups > THREADS) return 0;
  *tb = THREADS / *kgroups;
  const size_t bytes = ((size_t)16 * *reff * *kgroups * 4 + (size_t)*tb * 16 * *reff) * sizeof(float);
  return bytes <= 200 * 1024 ? bytes : 0;
}

template <typename T>
static cudaError_t launch_t(const FGeom &g, const void *x, const void *u, const void *bias, void *y, int sm_count,
                            cudaStream_t s, const char **detail) {
  int reff, kgroups, tb;
  const size_t smem = plan_smem(g, &reff, &kgroups, &tb);
  auto kern = fused23_smallc_kernel<T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { *detail = "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed"; return e; }
  }
  const long long n_groups = (g.T + tb - 1) / tb;
  const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / (smem + 1024)));
  const int grid = (int)std::min<long long>(n_groups, (long long)sm_count * per_sm);
  kern<<<grid, THREADS, smem, s>>>((const T *)x, (const T *)u, (T *)y, (const T *)bias, g, reff, kgroups, tb, n_groups);
  return cudaGetLastError();
}
}  // namespace smallc

// ---------------------------------------------------------------------------------------------------------
// filter transform for the fused layout: U[pos 16][k][q * Cp + c] = (G g_q G^T)[pos], g_q the (zero padded)
// 3x3 window of piece q.  Computed in fp32, rounded once.
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) fused_filter_kernel(const T *__restrict__ w, T *__restrict__ u,
                                                           const __grid_constant__ FGeom g) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)g.K * g.R) return;
  const int k = (int)(idx / g.R), r = (int)(idx % g.R);
  const int q = r / g.Cp, c = r - q * g.Cp;
  float a[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) a[i] = 0.f;
  if (c < g.C) {
    const FPiece pc = g.pieces[q];
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        const int kh = pc.ph_h + g.sH * (pc.st_h + i), kw = pc.ph_w + g.sW * (pc.st_w + j);
        if (kh < g.kH && kw < g.kW) {
          long long off;
          if (g.weight_layout == WINOCONV_W_KCRS)
            off = ((((long long)k * g.C + c) * g.kD + pc.kd) * g.kH + kh) * g.kW + kw;
          else
            off = ((((long long)pc.kd * g.kH + kh) * g.kW + kw) * g.C + c) * g.K + k;
          a[i * 3 + j] = Elem<T>::load(w + off);
        }
      }
  }
  float b[12], d[16];
#pragma unroll
  for (int i = 0; i < 3; ++i) Xf<2, 3>::g<1, 1>(&a[i * 3], &b[i * 4]);
#pragma unroll
  for (int j = 0; j < 4; ++j) Xf<2, 3>::g<4, 4>(&b[j], &d[j]);
  const long long pos_stride = (long long)g.K * g.R;
  T *dst = u + (long long)k * g.R + r;
#pragma unroll
  for (int p = 0; p < 16; ++p) Elem<T>::store(dst + p * pos_stride, d[p]);
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
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

template <typename T, bool VEC>
static cudaError_t launch_t(const FGeom &g, const CUtensorMap &map_u, const void *x, void *y, const void *bias,
                            int sm_count, uint32_t idesc, cudaStream_t s, const char **detail) {
  auto kern = fused23_kernel<T, VEC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) { *detail = "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed"; return e; }
  const long long n_mblocks = (g.T + BM - 1) / BM;
  const int n_nblocks = (g.K + BN - 1) / BN;
  if (n_mblocks * n_nblocks > 0x7fffffffLL) { *detail = "too many work items"; return cudaErrorInvalidConfiguration; }
  const int grid = (int)std::min<long long>(n_mblocks * n_nblocks, sm_count);
  kern<<<grid, N_THREADS, SMEM_BYTES, s>>>(map_u, (const T *)x, (T *)y, (const T *)bias, g, (int)n_mblocks, n_nblocks, idesc);
  return cudaGetLastError();
}

}  // namespace fused

cudaError_t read_and_clear_fused_error(cudaStream_t s, unsigned int *code) {
  unsigned int host = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&host, g_fused_error, sizeof(host), 0, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemcpyToSymbolAsync(g_fused_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  *code = host;
  return e;
}

cudaError_t launch_fused_filter_transform(const FGeom &g, int dtype, const void *w, void *u, cudaStream_t s) {
  const long long n = (long long)g.K * g.R;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == WINOCONV_F16)
    fused::fused_filter_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)w, (__half *)u, g);
  else
    fused::fused_filter_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)w, (__nv_bfloat16 *)u, g);
  return cudaGetLastError();
}

cudaError_t launch_fused_forward(const FGeom &g, int dtype, const void *x, const void *u, const void *bias, void *y,
                                 cudaStream_t s, const char **detail) {
  *detail = "";
  {
    int reff, kgroups, tb;
    if (fused::smallc::plan_smem(g, &reff, &kgroups, &tb) != 0) {   // few input channels: fp32 FMA variant
      int dev = 0, sm_count = 0;
      cudaError_t e = cudaGetDevice(&dev);
      if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) { *detail = "cudaDeviceGetAttribute(MultiProcessorCount) failed"; return e; }
      return dtype == WINOCONV_F16 ? fused::smallc::launch_t<__half>(g, x, u, bias, y, sm_count, s, detail)
                                   : fused::smallc::launch_t<__nv_bfloat16>(g, x, u, bias, y, sm_count, s, detail);
    }
  }
  fused::EncodeTiledFn enc = fused::get_encode_fn();
  if (!enc) { *detail = "cuTensorMapEncodeTiled unavailable"; return cudaErrorNotSupported; }
  CUtensorMap map_u;
  const cuuint64_t dims[3] = {(cuuint64_t)g.R, (cuuint64_t)g.K, 16u};
  const cuuint64_t strides[2] = {(cuuint64_t)g.R * 2ull, (cuuint64_t)g.R * 2ull * (cuuint64_t)g.K};
  const cuuint32_t box[3] = {(cuuint32_t)fused::BK, (cuuint32_t)fused::BN, 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUtensorMapDataType dt = dtype == WINOCONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (enc(&map_u, dt, 3, const_cast<void *>(u), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    *detail = "cuTensorMapEncodeTiled failed for the transformed filter";
    return cudaErrorInvalidValue;
  }
  int dev = 0, sm_count = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) { *detail = "cudaDeviceGetAttribute(MultiProcessorCount) failed"; return e; }
  const uint32_t fmt = dtype == WINOCONV_F16 ? 0u : 1u;
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(fused::BN >> 3) << 17) | ((uint32_t)(fused::BM >> 4) << 24);
  const bool vec = (g.C % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  if (dtype == WINOCONV_F16)
    return vec ? fused::launch_t<__half, true>(g, map_u, x, y, bias, sm_count, idesc, s, detail)
               : fused::launch_t<__half, false>(g, map_u, x, y, bias, sm_count, idesc, s, detail);
  return vec ? fused::launch_t<__nv_bfloat16, true>(g, map_u, x, y, bias, sm_count, idesc, s, detail)
             : fused::launch_t<__nv_bfloat16, false>(g, map_u, x, y, bias, sm_count, idesc, s, detail);
}

}  // namespace wino
