// Row-piece DWM forward for f16 / bf16, stride 1, on sm_100a: the kernel is decomposed the DWM way into
// 1 x 3 pieces -- along W every run of three taps is a Winograd F(2,3) window (zero taps where the kernel
// ends), along H (and depth) every tap is its own piece, for which F(m,1) is the identity.  All pieces write
// the same four Winograd positions of a tile of 1 x 2 outputs, so they are summed where the GEMM accumulates:
//
//     M[j][tile][k] = sum_{kd,kh,w} sum_c  V_w[row(tile) + kh][colpair(tile)][j][c] * U[kd][kh][w][j][k][c]
//     y[tile][0] = M0 + M1 + M2,   y[tile][1] = M1 - M2 - M3
//
// Why this shape on B200: with both MMA operands in shared memory a narrow accumulator (2-D F(2x2,3x3) needs 16
// positions, i.e. N = 32 columns each in the 512-column TMEM) is bound by the A-operand read, not by the tensor
// pipe.  Four positions leave N = 128, and the tap along H costs nothing to form: a 128-tile block is 8 (or 16)
// output rows x 16 (or 8) column pairs, the transformed slab holds all input rows of the block once, and tap kh
// is the same slab read through a descriptor that starts kh row-groups later.
//
// One persistent CTA per SM; per work item (tile block x 64/128 output channels):
//   warp 0       TMA: raw input patch (5-D box, zero fill = padding) per 32-channel slab
//   warps 1-8    F(2,3) along W on the patch: raw -> four [rows x 32] slabs, 64-byte swizzle, fence.proxy.async
//   warp 9       TMA: transformed-filter slabs of the current (kd, kh, window), four positions per stage
//   warp 10      tcgen05.mma (M = 128, N = BN, K = 16) issue + commits; TMEM alloc
//   warps 11-14  epilogue: tcgen05.ld, A^T along W, bias / ReLU / 2x2 max-pool (row partner by shuffle), 32-byte stores
// V and M never exist in global memory.  Every mbarrier wait is bounded and reports through the error word.
//
// Reference counterparts: the whole chain of src/base_conv_launchers.cu:338-381 (inputNorm2WinoTransform,
// cublas batched GEMM, outputWino2NormTransform, outputAggregate) and the piece table of
// src/base_conv_launchers.h:58-388, here with 1 x 3 pieces.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "wino_common.cuh"
#include "wino_launch.h"

namespace wino {

__device__ unsigned int g_row_error = 0;

#ifdef WINO_ROW_TRACE
// Development aid (not built by default): per-role accumulated wait clocks of CTA 0.
__device__ unsigned long long g_row_trace[32];
__device__ unsigned long long g_row_tl[10][256];     // event timeline of CTA 0: [role][event index] = clock64
#define TL(role, idx) do { if (blockIdx.x == 0 && (idx) < 256) g_row_tl[role][idx] = (unsigned long long)clock64(); } while (0)
#else
#define TL(role, idx) do { } while (0)
#endif

namespace rowf {

constexpr int BM = 128;            // tiles per block == TMEM lanes
constexpr int KC = 32;             // reduction slab (channels): 64-byte rows
constexpr int UMMA_K = 16;
constexpr int N_PROD = 256;
constexpr int N_THREADS = 480;     // 15 warps
constexpr long long WAIT_LIMIT_CLOCKS = 2000000000LL;

enum ErrCode : unsigned {
  ERR_RAW_EMPTY = 0x301, ERR_PROD_RAW = 0x302, ERR_PROD_A = 0x303, ERR_B_EMPTY = 0x304, ERR_MMA_ACC = 0x305,
  ERR_MMA_A = 0x306, ERR_MMA_B = 0x307, ERR_EPI = 0x308
};

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
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
// Polling wait (non-blocking test_wait) for the two threads on the MMA critical path.
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity, volatile unsigned *abort_word, unsigned code) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long start = clock64();
  unsigned spins = 0;
  while (!mbar_test_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (*abort_word != 0u) return false;
      if (clock64() - start > WAIT_LIMIT_CLOCKS) {
        *abort_word = code;
        atomicCAS(&g_row_error, 0u, code);
        return false;
      }
    }
  }
#ifdef WINO_ROW_TRACE
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) atomicAdd(&g_row_trace[code & 15u], (unsigned long long)(clock64() - start));
#endif
  return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile unsigned *abort_word, unsigned code,
                                          bool backoff = false) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (backoff) __nanosleep(200);     // roles with slack yield their issue slots to the MMA thread
    if (*abort_word != 0u) return false;
    if (clock64() - start > WAIT_LIMIT_CLOCKS) {
      *abort_word = code;
      atomicCAS(&g_row_error, 0u, code);
      return false;
    }
  }
#ifdef WINO_ROW_TRACE
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) atomicAdd(&g_row_trace[code & 15u], (unsigned long long)(clock64() - start));
#endif
  return true;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// reduction-major operand, 64-byte rows, SWIZZLE_64B: eight-row groups are 512 B apart
__device__ __forceinline__ uint64_t make_smem_desc_sw64(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(512 >> 4) << 32) | (1ull << 46) | (4ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same MMA with the descriptors given as (low word, high word): the high word is a constant of the layout,
// so the issuing thread only does 32-bit adds on the low words between MMAs.  (One thread issues every MMA of
// the CTA; with the descriptors rebuilt per instruction its dependent-issue latency, not the tensor pipe, set
// the pace -- about 150 clocks per MMA instead of 64.)
constexpr uint32_t DESC_HI_SW64 = (uint32_t)(512 >> 4) | (1u << 14) | (4u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ void umma_f16_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(DESC_HI_SW64), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

template <typename T> struct P2;
template <> struct P2<__half> {
  using V = __half2;
  static __device__ __forceinline__ V from(float a, float b) { return __floats2half2_rn(a, b); }
};
template <> struct P2<__nv_bfloat16> {
  using V = __nv_bfloat162;
  static __device__ __forceinline__ V from(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <typename T> struct __align__(16) V8 { typename P2<T>::V h[4]; };
template <typename T> __device__ __forceinline__ V8<T> v8_add(const V8<T> &a, const V8<T> &b) {
  V8<T> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.h[i] = __hadd2(a.h[i], b.h[i]);
  return r;
}
template <typename T> __device__ __forceinline__ V8<T> v8_sub(const V8<T> &a, const V8<T> &b) {
  V8<T> r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.h[i] = __hsub2(a.h[i], b.h[i]);
  return r;
}

// 16 consecutive output channels of one pixel: two 16-byte stores (K a multiple of 8) or element-wise.
template <typename T>
__device__ __forceinline__ void store16(T *dst, const float (&v)[16], int kbase, int K, bool vec_ok) {
  if (vec_ok) {
    typename P2<T>::V pk[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) pk[c] = P2<T>::from(v[2 * c], v[2 * c + 1]);
    *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(&pk[0]);
    if (kbase + 8 < K) *reinterpret_cast<uint4 *>(dst + 8) = *reinterpret_cast<const uint4 *>(&pk[4]);
  } else {
#pragma unroll
    for (int c = 0; c < 16; ++c)
      if (kbase + c < K) Elem<T>::store(dst + c, v[c]);
  }
}

// Shared-memory carve-up computed on the host and passed in (all offsets from the 1024-aligned base).
struct Smem {
  int raw_bytes, a_bytes, b_stage_bytes;   // one raw patch; one set of four slabs; one stage of four filter slabs
  int n_b_stages, n_a_bufs;
  int off_raw[2], off_a[2], off_b, off_bars;
  int total;
};

struct RGeom {
  int N, C, K;
  int Cp;                 // channels of the (padded) input the TMA map addresses
  int D, H, W, oD, oH, oW, yH, yW;
  int pD, pH, pW, kD, kH, kW;
  int PW;                 // F(2,3) windows along W: ceil(kW / 3)
  int RB, CBW;            // tile block: RB output rows x CBW column pairs, RB * CBW == 128
  int MB;                 // tile blocks per work item, stacked along H (they share every filter slab)
  int n_rb, n_cb;         // blocks per image plane
  int slab_rows;          // (MB * RB + kH - 1) * CBW
  int patch_h, patch_w;   // raw patch extents (pixels)
  int n_chunks;           // ceil(C / 32)
  int n_nblocks;
  long long n_items;
  unsigned epilogue;
  unsigned dbg;           // timing experiments only (WINOCONV_ROW_DBG): 1 no filter TMA, 2 no input TMA, 4 no transform, 8 no MMA, 16 no stores
};

template <typename T, int BN, int MB>
__global__ void __launch_bounds__(N_THREADS, 1) rowfused_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                 const __grid_constant__ CUtensorMap map_u,
                                                                 T *__restrict__ y, const T *__restrict__ bias,
                                                                 const __grid_constant__ RGeom g,
                                                                 const __grid_constant__ Smem sl, uint32_t idesc) {
  constexpr int ACC_COLS = MB * 4 * BN;                  // MB blocks x 4 positions x BN columns per buffer
  constexpr int ACC_BUFS = (ACC_COLS <= 256) ? 2 : 1;
  extern __shared__ uint8_t smem_raw_[];
  const uint32_t raw0 = smem_u32(smem_raw_);
  const uint32_t base = (raw0 + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw_ + (base - raw0);
  // barriers: raw_full[2] raw_empty[2] a_full[2] a_empty[2] b_full[8] b_empty[8] acc_full[2] acc_empty[2]
  const uint32_t bars = base + sl.off_bars;
  auto raw_full = [&](int i) { return bars + 8u * i; };
  auto raw_empty = [&](int i) { return bars + 8u * (2 + i); };
  auto a_full = [&](int i) { return bars + 8u * (4 + i); };
  auto a_empty = [&](int i) { return bars + 8u * (6 + i); };
  auto b_full = [&](int i) { return bars + 8u * (8 + i); };
  auto b_empty = [&](int i) { return bars + 8u * (16 + i); };
  auto acc_full = [&](int i) { return bars + 8u * (24 + i); };
  auto acc_empty = [&](int i) { return bars + 8u * (26 + i); };
  volatile unsigned *abort_word = reinterpret_cast<volatile unsigned *>(base_ptr + sl.off_bars + 256);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + sl.off_bars + 260);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef WINO_ROW_TRACE
  const long long trace_kernel_t0 = clock64();
#endif
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(raw_full(i), 1);
      mbar_init(raw_empty(i), N_PROD);
      mbar_init(a_full(i), N_PROD);
      mbar_init(a_empty(i), 1);
      mbar_init(acc_full(i), 1);
      mbar_init(acc_empty(i), 128);
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(b_full(i), 1);
      mbar_init(b_empty(i), 1);
    }
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 10) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // item -> (n, od, rb, cb, nb); the channel block is the fastest index so consecutive CTAs share a patch
  auto decode = [&](long long item, int &n, int &od, int &rb, int &cb, int &nb) {
    nb = (int)(item % g.n_nblocks); item /= g.n_nblocks;
    cb = (int)(item % g.n_cb); item /= g.n_cb;
    rb = (int)(item % g.n_rb); item /= g.n_rb;
    od = (int)(item % g.oD); item /= g.oD;
    n = (int)item;
  };
  const int steps_per_item = g.kD * g.n_chunks;          // raw patches per item
  // CTAs walk the channel slabs in rotated order so that they do not all ask L2 for the same filter slab at once
  const int rot = (g.dbg & 256u) ? 0 : (int)(blockIdx.x % (unsigned)g.n_chunks);
  // When one channel block covers K and a whole item's filter slabs fit the stage ring, they are loaded once and
  // stay: stage index = slab position within the item, no refills.
  const bool b_resident = g.n_nblocks == 1 && steps_per_item * g.PW * g.kH <= sl.n_b_stages && !(g.dbg & 512u);

  if (warp == 0) {
    // ---------------------------------------------------------------- raw input patches
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (long long item = blockIdx.x; item < g.n_items && alive; item += gridDim.x) {
        int n, od, rb, cb, nb;
        decode(item, n, od, rb, cb, nb);
        for (int kd = 0; kd < g.kD && alive; ++kd)
          for (int ch = 0; ch < g.n_chunks; ++ch) {
            const int s = it & 1;
            if (!mbar_wait(raw_empty(s), ((it >> 1) & 1u) ^ 1u, abort_word, ERR_RAW_EMPTY, (g.dbg & 32u) != 0)) { alive = false; break; }
            if (g.dbg & 2u) { mbar_arrive(raw_full(s)); ++it; continue; }
            mbar_expect_tx(raw_full(s), (uint32_t)sl.raw_bytes);
            tma_load_5d(base + sl.off_raw[s], &map_x, raw_full(s), ((ch + rot) % g.n_chunks) * KC, cb * g.CBW * 2 - g.pW, rb * (MB * g.RB) - g.pH,
                        od + kd - g.pD, n);
            ++it;
          }
      }
    }
  } else if (warp <= 8) {
    // ---------------------------------------------------------------- F(2,3) along W: raw patch -> four slabs
    const int ptid = threadIdx.x - 32;                 // 0..255
    const int v = ptid & 3;                            // 16-byte vector of the 32-channel slab
    const int n_tasks = g.slab_rows;                   // one task = one slab row (input row, column pair) x one vector
    uint32_t it_raw = 0, it_a = 0;
    bool alive = true;
    for (long long item = blockIdx.x; item < g.n_items && alive; item += gridDim.x) {
      for (int step = 0; step < steps_per_item && alive; ++step) {
        const int rs = it_raw & 1;
        if (!((g.dbg & 128u) ? mbar_poll(raw_full(rs), (it_raw >> 1) & 1u, abort_word, ERR_PROD_RAW) : mbar_wait(raw_full(rs), (it_raw >> 1) & 1u, abort_word, ERR_PROD_RAW, (g.dbg & 32u) != 0))) { alive = false; break; }
        if (ptid == 0) TL(8, it_raw);
        const uint8_t *raw = base_ptr + sl.off_raw[rs];
        for (int w = 0; w < g.PW && alive; ++w) {
          const int as = (int)(it_a % (uint32_t)sl.n_a_bufs);
          if (!((g.dbg & 128u) ? mbar_poll(a_empty(as), ((it_a / (uint32_t)sl.n_a_bufs) & 1u) ^ 1u, abort_word, ERR_PROD_A) : mbar_wait(a_empty(as), ((it_a / (uint32_t)sl.n_a_bufs) & 1u) ^ 1u, abort_word, ERR_PROD_A, (g.dbg & 32u) != 0))) { alive = false; break; }
          if (ptid == 0) TL(4, it_a);
          uint8_t *slab = base_ptr + sl.off_a[as];
          const int slab_bytes = g.slab_rows * 64;
          for (int row = ptid >> 2; row < ((g.dbg & 4u) ? 0 : n_tasks); row += N_PROD / 4) {
            const int ir = row / g.CBW, cp = row - ir * g.CBW;
            const uint8_t *src = raw + ((size_t)(ir * g.patch_w + 2 * cp + 3 * w) * KC + v * 8) * 2;
            V8<T> d0, d1, d2, d3;
            *reinterpret_cast<uint4 *>(&d0) = *reinterpret_cast<const uint4 *>(src);
            *reinterpret_cast<uint4 *>(&d1) = *reinterpret_cast<const uint4 *>(src + KC * 2);
            *reinterpret_cast<uint4 *>(&d2) = *reinterpret_cast<const uint4 *>(src + 2 * KC * 2);
            *reinterpret_cast<uint4 *>(&d3) = *reinterpret_cast<const uint4 *>(src + 3 * KC * 2);
            const V8<T> o0 = v8_sub<T>(d0, d2), o1 = v8_add<T>(d1, d2), o2 = v8_sub<T>(d2, d1), o3 = v8_sub<T>(d1, d3);
            // 64-byte swizzle: 16-byte chunk index XOR ((row >> 1) & 3)
            const uint32_t off = (uint32_t)row * 64u + (uint32_t)((v ^ ((row >> 1) & 3)) << 4);
            *reinterpret_cast<uint4 *>(slab + off) = *reinterpret_cast<const uint4 *>(&o0);
            *reinterpret_cast<uint4 *>(slab + slab_bytes + off) = *reinterpret_cast<const uint4 *>(&o1);
            *reinterpret_cast<uint4 *>(slab + 2 * slab_bytes + off) = *reinterpret_cast<const uint4 *>(&o2);
            *reinterpret_cast<uint4 *>(slab + 3 * slab_bytes + off) = *reinterpret_cast<const uint4 *>(&o3);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive(a_full(as));
          if (ptid == 0) TL(5, it_a);
          ++it_a;
        }
        if (alive) mbar_arrive(raw_empty(rs));     // all windows of this patch are transformed
        ++it_raw;
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- transformed-filter slabs
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      const int nbs = sl.n_b_stages;
      for (long long item = blockIdx.x; item < g.n_items && alive; item += gridDim.x) {
        int n, od, rb, cb, nb;
        decode(item, n, od, rb, cb, nb);
        if (b_resident && item != (long long)blockIdx.x) break;   // every slab of the filter is already in shared memory
        for (int kd = 0; kd < g.kD && alive; ++kd)
          for (int ch = 0; ch < g.n_chunks && alive; ++ch)
            for (int w = 0; w < g.PW && alive; ++w)
              for (int kh = 0; kh < g.kH; ++kh) {
                const int s = it % nbs;
                if (!((g.dbg & 64u) ? mbar_poll(b_empty(s), ((it / nbs) & 1u) ^ 1u, abort_word, ERR_B_EMPTY) : mbar_wait(b_empty(s), ((it / nbs) & 1u) ^ 1u, abort_word, ERR_B_EMPTY, (g.dbg & 32u) != 0))) { alive = false; break; }
                TL(2, it);
                if (g.dbg & 1u) { mbar_arrive(b_full(s)); ++it; continue; }
                mbar_expect_tx(b_full(s), (uint32_t)sl.b_stage_bytes);
                const int slab0 = ((kd * g.kH + kh) * g.PW + w) * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  tma_load_3d(base + sl.off_b + s * sl.b_stage_bytes + j * (BN * 64), &map_u, b_full(s), ((ch + rot) % g.n_chunks) * KC, nb * BN, slab0 + j);
                TL(3, it);
                ++it;
              }
      }
      if (*abort_word != 0u) {
        const long long start = clock64();
        while (clock64() - start < 2000000LL) { }
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
#ifdef WINO_ROW_TRACE
      if (blockIdx.x == 0) {   // latency of an empty tcgen05.commit -> mbarrier flip, and of a plain arrive
        const uint32_t tb = bars + 8u * 28;
        mbar_init(tb, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int rep = 0; rep < 4; ++rep) {
          const long long t0 = clock64();
          umma_commit(tb);
          while (!mbar_test_wait(tb, (uint32_t)(rep & 1))) { }
          g_row_trace[24] += (unsigned long long)(clock64() - t0);
        }
        for (int rep = 4; rep < 8; ++rep) {
          const long long t0 = clock64();
          mbar_arrive(tb);
          while (!mbar_test_wait(tb, (uint32_t)(rep & 1))) { }
          g_row_trace[25] += (unsigned long long)(clock64() - t0);
        }
      }
#endif
      uint32_t it_a = 0, it_b = 0, n_done = 0;
      bool alive = true;
#ifdef WINO_ROW_TRACE
      // LAP(k): clocks since the previous LAP are charged to segment k (register accumulators, written once)
      long long lap_t = clock64();
      unsigned long long lap_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define LAP(k) do { const long long now_ = clock64(); lap_acc[k] += (unsigned long long)(now_ - lap_t); lap_t = now_; } while (0)
#else
#define LAP(k) do { } while (0)
#endif
      const int nbs = sl.n_b_stages;
      const uint32_t slab16 = (uint32_t)(g.slab_rows * 64 / 16);
      static_assert(KC / UMMA_K == 2, "two K = 16 steps per slab");
      for (long long item = blockIdx.x; item < g.n_items && alive; item += gridDim.x, ++n_done) {
        const int ab = (ACC_BUFS == 2) ? (int)(n_done & 1u) : 0;
        const uint32_t use = (ACC_BUFS == 2) ? (n_done >> 1) : n_done;
        LAP(6);
        if (!mbar_wait(acc_empty(ab), (use & 1u) ^ 1u, abort_word, ERR_MMA_ACC)) { alive = false; break; }
        LAP(7);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + (uint32_t)(ab * ACC_COLS);
        bool first = true;
        for (int step = 0; step < steps_per_item && alive; ++step) {
          // a slab with at most 16 real channels (few-channel input, or the tail of C) needs one K = 16 step only
          const bool k2 = g.Cp - ((step + rot) % g.n_chunks) * KC > UMMA_K;
          for (int w = 0; w < g.PW && alive; ++w) {
            const int as = (int)(it_a % (uint32_t)sl.n_a_bufs);
            if (!((g.dbg & 64u) ? mbar_poll(a_full(as), (it_a / (uint32_t)sl.n_a_bufs) & 1u, abort_word, ERR_MMA_A) : mbar_wait(a_full(as), (it_a / (uint32_t)sl.n_a_bufs) & 1u, abort_word, ERR_MMA_A))) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            TL(9, it_a);
            const uint32_t a_lo0 = desc_lo(base + sl.off_a[as]);
            for (int kh = 0; kh < g.kH; ++kh) {
              LAP(0);
              const int bs = b_resident ? (int)(it_b % (uint32_t)(steps_per_item * g.PW * g.kH)) : (int)(it_b % nbs);
              if (!(b_resident && n_done > 0))
                if (!((g.dbg & 64u) ? mbar_poll(b_full(bs), b_resident ? 0u : ((it_b / nbs) & 1u), abort_word, ERR_MMA_B) : mbar_wait(b_full(bs), b_resident ? 0u : ((it_b / nbs) & 1u), abort_word, ERR_MMA_B))) { alive = false; break; }
              LAP(1); TL(0, it_b);
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              const uint32_t b_lo0 = desc_lo(base + sl.off_b + bs * sl.b_stage_bytes);
              const uint32_t a_lo_kh = a_lo0 + (uint32_t)(kh * g.CBW * 4);      // 64-byte rows = 4 descriptor units
              const uint32_t acc0 = first ? 0u : 1u;
              LAP(2);
              if (!(g.dbg & 8u)) {
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                  uint32_t a_lo = a_lo_kh + (uint32_t)(mb * BM * 4);            // block mb starts RB * CBW = 128 rows later
                  uint32_t b_lo = b_lo0;
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const uint32_t d_col = acc + (uint32_t)((mb * 4 + j) * BN);
                    umma_f16_lohi(d_col, a_lo, b_lo, idesc, acc0);
                    if (k2) umma_f16_lohi(d_col, a_lo + 2u, b_lo + 2u, idesc, 1u);   // second K = 16 step: 32 bytes further
                    a_lo += slab16;
                    b_lo += (uint32_t)(BN * 64 / 16);
                  }
                }
              }
              first = false;
              LAP(3); TL(1, it_b);
              if (!b_resident) umma_commit(b_empty(bs));
              LAP(4);
              ++it_b;
            }
            umma_commit(a_empty(as));
            ++it_a;
          }
        }
        umma_commit(acc_full(ab));
        LAP(5);
      }
#ifdef WINO_ROW_TRACE
      if (blockIdx.x == 0) for (int k = 0; k < 8; ++k) g_row_trace[16 + k] += lap_acc[k];
#endif
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int qd = warp & 3;                           // TMEM lane quarter
    const int row = qd * 32 + lane;                    // tile of the block: (out row, column pair)
    const int tr = row / g.CBW, tcp = row - tr * g.CBW;
    const bool relu = (g.epilogue & WINOCONV_EPI_RELU) != 0;
    const bool has_bias = (g.epilogue & WINOCONV_EPI_BIAS) != 0;
    const bool pool = (g.epilogue & WINOCONV_EPI_POOL2) != 0;
    const bool vec_ok = (g.K % 8) == 0;
    uint32_t n_done = 0;
    bool alive = true;
    for (long long item = blockIdx.x; item < g.n_items && alive; item += gridDim.x, ++n_done) {
      int n, od, rb, cb, nb;
      decode(item, n, od, rb, cb, nb);
      const int ab = (ACC_BUFS == 2) ? (int)(n_done & 1u) : 0;
      const uint32_t use = (ACC_BUFS == 2) ? (n_done >> 1) : n_done;
      unsigned got = 0;
      if (lane == 0) got = mbar_wait(acc_full(ab), use & 1u, abort_word, ERR_EPI, (g.dbg & 32u) != 0) ? 1u : 0u;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got == 0u) { alive = false; break; }
      if (warp == 11 && lane == 0) TL(6, n_done);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int ow = (cb * g.CBW + tcp) * 2;
#pragma unroll 1
      for (int mb = 0; mb < MB; ++mb) {
      const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(ab * ACC_COLS + mb * 4 * BN);
      const int oh = (rb * MB + mb) * g.RB + tr;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t m0[16], m1[16], m2[16], m3[16];
        tmem_ld_x16(t_lane + (uint32_t)(0 * BN + c0), m0);
        tmem_ld_x16(t_lane + (uint32_t)(1 * BN + c0), m1);
        tmem_ld_x16(t_lane + (uint32_t)(2 * BN + c0), m2);
        tmem_ld_x16(t_lane + (uint32_t)(3 * BN + c0), m3);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 16 >= BN && mb == MB - 1) {   // last columns are in registers: hand the accumulator back
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(acc_empty(ab));
          if (warp == 11 && lane == 0) TL(7, n_done);
        }
        const int kbase = nb * BN + c0;
        float y0[16], y1[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float a0 = __uint_as_float(m0[c]), a1 = __uint_as_float(m1[c]), a2 = __uint_as_float(m2[c]), a3 = __uint_as_float(m3[c]);
          float bv = 0.f;
          if (has_bias && kbase + c < g.K) bv = Elem<T>::load(bias + kbase + c);
          y0[c] = a0 + a1 + a2 + bv;
          y1[c] = a1 - a2 - a3 + bv;
        }
        if (pool) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float mx = fmaxf(y0[c], y1[c]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, g.CBW));   // the other output row of the 2x2 window
            y0[c] = relu ? fmaxf(mx, 0.f) : mx;
          }
          const int ph = oh >> 1, pw = ow >> 1;
          if ((tr & 1) == 0 && ph < g.yH && pw < g.yW && kbase < g.K && !(g.dbg & 16u)) {
            T *dst = y + ((((long long)n * g.oD + od) * g.yH + ph) * g.yW + pw) * g.K + kbase;
            store16<T>(dst, y0, kbase, g.K, vec_ok);
          }
        } else {
          if (relu) {
#pragma unroll
            for (int c = 0; c < 16; ++c) { y0[c] = fmaxf(y0[c], 0.f); y1[c] = fmaxf(y1[c], 0.f); }
          }
          if (oh < g.oH && kbase < g.K && !(g.dbg & 16u)) {
            T *dst = y + ((((long long)n * g.oD + od) * g.oH + oh) * g.oW + ow) * g.K + kbase;
            if (ow < g.oW) store16<T>(dst, y0, kbase, g.K, vec_ok);
            if (ow + 1 < g.oW) store16<T>(dst + g.K, y1, kbase, g.K, vec_ok);
          }
        }
      }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
#ifdef WINO_ROW_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    g_row_trace[0] += (unsigned long long)(clock64() - trace_kernel_t0);
    g_row_trace[15] += (unsigned long long)((g.n_items + gridDim.x - 1) / gridDim.x);
  }
#endif
  if (warp == 10) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// U[slab][k][c], slab = ((kd * kH + kh) * PW + w) * 4 + j:  G (3 taps of window w, zero padded) along W.
template <typename T>
__global__ void __launch_bounds__(256) rowfused_filter_kernel(const T *__restrict__ wgt, T *__restrict__ u, int C, int Cp,
                                                              int K, int kD, int kH, int kW, int PW, int layout) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long per_k = (long long)kD * kH * PW * Cp;
  if (idx >= per_k * K) return;
  const int k = (int)(idx / per_k);
  long long rem = idx - (long long)k * per_k;
  const int c = (int)(rem % Cp); rem /= Cp;
  const int w = (int)(rem % PW); rem /= PW;
  const int kh = (int)(rem % kH);
  const int kd = (int)(rem / kH);
  float a[3] = {0.f, 0.f, 0.f}, o[4];
  if (c < C) {
#pragma unroll
    for (int t = 0; t < 3; ++t) {
      const int kw = 3 * w + t;
      if (kw < kW) {
        const long long off = layout == WINOCONV_W_KCRS ? ((((long long)k * C + c) * kD + kd) * kH + kh) * kW + kw
                                                        : ((((long long)kd * kH + kh) * kW + kw) * C + c) * K + k;
        a[t] = Elem<T>::load(wgt + off);
      }
    }
  }
  Xf<2, 3>::g<1, 1>(a, o);
  const long long slab0 = (((long long)kd * kH + kh) * PW + w) * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) Elem<T>::store(u + ((slab0 + j) * K + k) * Cp + c, o[j]);
}

// zero-pads the channel dimension to a multiple of 8 so the input can be addressed by TMA; one thread writes one
// 16-byte group of eight channels
template <typename T>
__global__ void __launch_bounds__(256) pad_channels_kernel(const T *__restrict__ x, T *__restrict__ xp, long long pixels,
                                                           int C, int Cp) {
  const int groups = Cp / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= pixels * groups) return;
  const long long px = idx / groups;
  const int c0 = (int)(idx - px * groups) * 8;
  __align__(16) T v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = (c0 + i < C) ? x[px * C + c0 + i] : T(0.f);
  *reinterpret_cast<uint4 *>(xp + px * Cp + c0) = *reinterpret_cast<const uint4 *>(v);
}

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

}  // namespace rowf

// Fills the geometry of the row-piece kernel for this convolution; returns false when it does not apply
// (stride 2, kernel taller than 7, or a patch / slab that does not fit shared memory).
bool rowfused_plan(const RowDesc &d, RowPlan *out) {
  using namespace rowf;
  if (d.sD != 1 || d.sH != 1 || d.sW != 1) return false;
  if (d.kH > 7 || d.kW > 10 || d.kD > 10) return false;
  RowPlan p;
  const int Cp = (d.C + 7) / 8 * 8;
  p.Cp = Cp;
  p.PW = (d.kW + 2) / 3;
  // Work item: MB tile blocks stacked along H x BN output channels, MB * BN = 128 (the 512 TMEM columns hold
  // MB x 4 positions x BN).  Two blocks x 64 channels halve the filter bytes streamed per multiply-add, which is
  // what the kernel runs out of first; one block x 128 channels is kept for images too short for two blocks.
  // WINOCONV_ROW_MB=1|2 forces the choice (tuning).
  const int ncp = (d.oW + 1) / 2;
  auto padded = [&](int rows_item, int cbw) {
    return (long long)((d.oH + rows_item - 1) / rows_item) * rows_item * ((ncp + cbw - 1) / cbw) * cbw;
  };
  int best_mb = 0, best_cbw = 0;
  long long best = -1;
  static const int forced_mb = [] { const char *v = getenv("WINOCONV_ROW_MB"); return v && *v ? atoi(v) : 0; }();
  for (int mb = 2; mb >= 1; --mb) {
    if (forced_mb && mb != forced_mb) continue;
    for (int cbw : {16, 8}) {
      const long long vol = padded(mb * (128 / cbw), cbw);
      // prefer two blocks unless that pads more than 15 % over the best one-block shape
      const long long score = mb == 2 ? vol * 100 : vol * 115;
      if (best < 0 || score < best) { best = score; best_mb = mb; best_cbw = cbw; }
    }
  }
  p.MB = best_mb;
  p.BN = (p.MB == 2 || d.K <= 64) ? 64 : 128;
  p.CBW = best_cbw;
  p.RB = 128 / p.CBW;
  p.n_rb = (d.oH + p.MB * p.RB - 1) / (p.MB * p.RB);
  p.n_cb = (ncp + p.CBW - 1) / p.CBW;
  p.slab_rows = (p.MB * p.RB + d.kH - 1) * p.CBW;
  p.patch_h = p.MB * p.RB + d.kH - 1;
  p.patch_w = 2 * p.CBW + 3 * p.PW - 1;
  p.n_chunks = (Cp + KC - 1) / KC;
  p.n_nblocks = (d.K + p.BN - 1) / p.BN;
  p.slabs = d.kD * d.kH * p.PW * 4;
  p.filter_elems = (long long)p.slabs * d.K * Cp;
  p.n_items = (long long)d.N * d.oD * p.n_rb * p.n_cb * p.n_nblocks;
  if (p.patch_w > 256 || p.patch_h > 256) return false;
  // shared memory: 2 raw patches, 2 slab sets (1 if two do not leave room for 3 filter stages), then as many
  // filter stages as fit (2..8)
  const int raw_bytes = ((p.patch_h * p.patch_w * KC * 2 + 127) / 128) * 128;
  const int a_bytes = ((4 * p.slab_rows * 64 + 1023) / 1024) * 1024;
  const int b_stage = 4 * p.BN * 64;
  const int budget = 227 * 1024;
  int n_a = 2;
  int fixed = 2 * raw_bytes + n_a * a_bytes + 1024 /*bars*/ + 1024 /*align*/;
  if ((budget - fixed) / b_stage < 3) {
    n_a = 1;
    fixed = 2 * raw_bytes + n_a * a_bytes + 2048;
  }
  int nb = (budget - fixed) / b_stage;
  if (nb < 2) return false;
  if (nb > 8) nb = 8;
  p.n_a_bufs = n_a;
  p.raw_bytes = raw_bytes; p.a_bytes = a_bytes; p.b_stage_bytes = b_stage; p.n_b_stages = nb;
  p.smem_total = fixed + nb * b_stage;
  *out = p;
  return true;
}

cudaError_t launch_rowfused_filter_transform(const RowDesc &d, const RowPlan &p, int dtype, const void *w, void *u, cudaStream_t s) {
  const long long n = (long long)d.kD * d.kH * p.PW * p.Cp * d.K;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == WINOCONV_F16)
    rowf::rowfused_filter_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)w, (__half *)u, d.C, p.Cp, d.K, d.kD, d.kH, d.kW, p.PW, d.weight_layout);
  else
    rowf::rowfused_filter_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)w, (__nv_bfloat16 *)u, d.C, p.Cp, d.K, d.kD, d.kH, d.kW, p.PW, d.weight_layout);
  return cudaGetLastError();
}

template <typename T, int BN, int MB>
static cudaError_t launch_rf(const RowDesc &d, const RowPlan &p, const CUtensorMap &mx, const CUtensorMap &mu, void *y,
                             const void *bias, int sm_count, uint32_t idesc, cudaStream_t s, const char **detail) {
  using namespace rowf;
  auto kern = rowfused_kernel<T, BN, MB>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_total);
  if (e != cudaSuccess) { *detail = "cudaFuncSetAttribute(MaxDynamicSharedMemorySize) failed"; return e; }
  RGeom g;
  g.N = d.N; g.C = d.C; g.K = d.K; g.Cp = p.Cp; g.D = d.D; g.H = d.H; g.W = d.W; g.oD = d.oD; g.oH = d.oH; g.oW = d.oW;
  g.yH = d.yH; g.yW = d.yW; g.pD = d.pD; g.pH = d.pH; g.pW = d.pW; g.kD = d.kD; g.kH = d.kH; g.kW = d.kW;
  g.PW = p.PW; g.RB = p.RB; g.CBW = p.CBW; g.MB = p.MB; g.n_rb = p.n_rb; g.n_cb = p.n_cb; g.slab_rows = p.slab_rows;
  g.patch_h = p.patch_h; g.patch_w = p.patch_w; g.n_chunks = p.n_chunks; g.n_nblocks = p.n_nblocks;
  g.n_items = p.n_items; g.epilogue = d.epilogue;
  static const unsigned dbg = [] { const char *v = getenv("WINOCONV_ROW_DBG"); return v && *v ? (unsigned)atoi(v) : 0u; }();
  g.dbg = dbg;
  Smem sl;
  sl.raw_bytes = p.patch_h * p.patch_w * KC * 2;   // bytes the TMA box delivers
  sl.a_bytes = p.a_bytes; sl.b_stage_bytes = p.b_stage_bytes; sl.n_b_stages = p.n_b_stages;
  sl.n_a_bufs = p.n_a_bufs;
  sl.off_a[0] = 0; sl.off_a[1] = p.n_a_bufs == 2 ? p.a_bytes : 0;  // slabs first: 1024-byte aligned
  sl.off_b = p.n_a_bufs * p.a_bytes;                               // filter stages: multiples of 1024
  sl.off_raw[0] = sl.off_b + p.n_b_stages * p.b_stage_bytes;
  sl.off_raw[1] = sl.off_raw[0] + p.raw_bytes;
  sl.off_bars = sl.off_raw[1] + p.raw_bytes;
  sl.total = p.smem_total;
  const int grid = (int)std::min<long long>(p.n_items, sm_count);
  kern<<<grid, N_THREADS, p.smem_total, s>>>(mx, mu, (T *)y, (const T *)bias, g, sl, idesc);
  return cudaGetLastError();
}

cudaError_t launch_rowfused_forward(const RowDesc &d, const RowPlan &p, int dtype, const void *x, const void *u,
                                    const void *bias, void *y, void *pad_ws, cudaStream_t s, const char **detail) {
  using namespace rowf;
  *detail = "";
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { *detail = "cuTensorMapEncodeTiled unavailable"; return cudaErrorNotSupported; }
  const void *xin = x;
  if (p.Cp != d.C) {   // channels not a multiple of 8: TMA needs 16-byte pixel strides, so pad into scratch first
    if (!pad_ws) { *detail = "channel padding scratch missing"; return cudaErrorInvalidValue; }
    const long long pixels = (long long)d.N * d.D * d.H * d.W;
    const unsigned blocks = (unsigned)((pixels * (p.Cp / 8) + 255) / 256);
    if (dtype == WINOCONV_F16)
      pad_channels_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)x, (__half *)pad_ws, pixels, d.C, p.Cp);
    else
      pad_channels_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)pad_ws, pixels, d.C, p.Cp);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { *detail = "channel padding launch failed"; return e; }
    xin = pad_ws;
  }
  const CUtensorMapDataType dt = dtype == WINOCONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap mx, mu;
  {
    const cuuint64_t dims[5] = {(cuuint64_t)p.Cp, (cuuint64_t)d.W, (cuuint64_t)d.H, (cuuint64_t)d.D, (cuuint64_t)d.N};
    const cuuint64_t st[4] = {(cuuint64_t)p.Cp * 2ull, (cuuint64_t)p.Cp * 2ull * d.W, (cuuint64_t)p.Cp * 2ull * d.W * d.H,
                              (cuuint64_t)p.Cp * 2ull * d.W * d.H * d.D};
    const cuuint32_t box[5] = {(cuuint32_t)KC, (cuuint32_t)p.patch_w, (cuuint32_t)p.patch_h, 1u, 1u};
    const cuuint32_t es[5] = {1u, 1u, 1u, 1u, 1u};
    if (enc(&mx, dt, 5, const_cast<void *>(xin), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *detail = "cuTensorMapEncodeTiled failed for the input";
      return cudaErrorInvalidValue;
    }
  }
  {
    const cuuint64_t dims[3] = {(cuuint64_t)p.Cp, (cuuint64_t)d.K, (cuuint64_t)p.slabs};
    const cuuint64_t st[2] = {(cuuint64_t)p.Cp * 2ull, (cuuint64_t)p.Cp * 2ull * d.K};
    const cuuint32_t box[3] = {(cuuint32_t)KC, (cuuint32_t)p.BN, 1u};
    const cuuint32_t es[3] = {1u, 1u, 1u};
    if (enc(&mu, dt, 3, const_cast<void *>(u), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      *detail = "cuTensorMapEncodeTiled failed for the transformed filter";
      return cudaErrorInvalidValue;
    }
  }
  int dev = 0, sm_count = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) { *detail = "cudaDeviceGetAttribute(MultiProcessorCount) failed"; return e; }
  const uint32_t fmt = dtype == WINOCONV_F16 ? 0u : 1u;
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  if (dtype == WINOCONV_F16) {
    if (p.MB == 2) return launch_rf<__half, 64, 2>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail);
    return p.BN == 64 ? launch_rf<__half, 64, 1>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail)
                      : launch_rf<__half, 128, 1>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail);
  }
  if (p.MB == 2) return launch_rf<__nv_bfloat16, 64, 2>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail);
  return p.BN == 64 ? launch_rf<__nv_bfloat16, 64, 1>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail)
                    : launch_rf<__nv_bfloat16, 128, 1>(d, p, mx, mu, y, bias, sm_count, idesc, s, detail);
}

#ifdef WINO_ROW_TRACE
extern "C" __attribute__((visibility("default"))) int winoconv_debug_row_timeline(unsigned long long *out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(out, g_row_tl, sizeof(unsigned long long) * 10 * 256);
}
extern "C" __attribute__((visibility("default"))) int winoconv_debug_row_trace(unsigned long long *out, int clear) {
  cudaDeviceSynchronize();
  cudaError_t e = cudaMemcpyFromSymbol(out, g_row_trace, sizeof(unsigned long long) * 32);
  if (e == cudaSuccess && clear) {
    unsigned long long z[32] = {};
    e = cudaMemcpyToSymbol(g_row_trace, z, sizeof(z));
  }
  return (int)e;
}
#endif

cudaError_t read_and_clear_row_error(cudaStream_t s, unsigned int *code) {
  unsigned int host = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&host, g_row_error, sizeof(host), 0, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemcpyToSymbolAsync(g_row_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  *code = host;
  return e;
}

}  // namespace wino
