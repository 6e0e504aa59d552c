// Importance scores of a prefilled layer straight from the observation window's queries and the
// layer's keys, without the [H_q, W, T] attention weights ever reaching memory.
//
// Replaces the scoring step of the reference's prefill (obkv_fast.py:1443-1466): attention weights
// of the last W query positions over all T keys (matmul in the model's 16-bit type, scaled, causal
// mask, softmax), then _score_one_layer (:854-896): token score [H_kv][T] = sum of the weights
// over the head's g query heads and the W positions, channel score [H_kv][128] = mean(q^2) *
// mean_t(k^2).  The reference materialises the weights (2 bytes x H_q x W x T) and reads them
// back; here a tile of scores lives in tensor memory and registers only.
//
// The contraction runs on the fifth-generation tensor cores.  A CTA belongs to one KV head and
// streams every P-th 128-key tile of it (P CTAs per head, about two CTAs per SM in all):
//   * the head's g*W query rows arrive once, the key tiles through a ring of two buffers, all in
//     the tensor cores' K-major layout with 128-byte swizzle: tiled TMA copies through two tensor
//     maps when the strides allow it, plain 16-byte loads with the same swizzle otherwise;
//   * thread 0 issues eight tcgen05.mma (K = 16 channels each) per tile into one of two fp32
//     accumulators in tensor memory and a tcgen05.commit onto an mbarrier; the products of tile
//     n+1 and the copies of tile n+2 run while the 8 warps work through tile n;
//   * the warps read the accumulator back with tcgen05.ld, 32 columns of ONE accumulator row per
//     thread at a time.
// Three launches per layer:
//   obs_stream_kernel<.,0>  S = Q.K^T (accumulator row = query row): scores rounded as the
//                           reference's 16-bit matmul and scaling round them, masked; a thread
//                           keeps its row's running maximum and sum of exponentials over the
//                           CTA's tiles (no exchange between threads) and the tile's k^2.
//   obs_reduce_kernel       the rows' maxima and sums over the CTAs of a head.
//   obs_stream_kernel<.,1>  S^T = K.Q^T (accumulator row = key): the same scores again, p =
//                           exp(s - M) / L rounded to the 16-bit type and summed over the query
//                           rows inside the thread: the token scores.  One more CTA per head
//                           turns the k^2 sums and the queries into the channel score meanwhile.
// The keys are read twice (the second time mostly from L2); sums run in a fixed order.
//
// Only thread 0 waits on mbarriers, every such wait is bounded, and the other threads meet it at
// CTA barriers.  A wait that runs out sets a bit in the status word (the last word of the scratch
// buffer: 1 = operands did not arrive, 2 = products did not complete); the kernel still frees its
// tensor memory and returns, and the results are invalid.
#include <cuda.h>   // CUtensorMap and its enums (the encoder itself is looked up through the runtime)

#include <algorithm>
#include <cstring>
#include <type_traits>

#include "rdkv_common.cuh"

namespace rdkv {

constexpr int OBS_THREADS = 256;                 // 8 warps: warp w reads accumulator rows 32*(w&3).., column half w>>2
constexpr int OBS_KEYS = 128;                    // keys per tile
constexpr int OBS_ROWS = 128;                    // query rows per block of the first pass (M of its MMAs)
constexpr int OBS_MAX_ROWS = 256;                // (query head, position) pairs per KV head: two blocks
constexpr int OBS_PANEL = 128 * 128;             // bytes: 128 rows of 64 16-bit channels, 128 bytes a row
constexpr int OBS_BLOCK = 2 * OBS_PANEL;         // a 128-row operand: channels 0-63, then channels 64-127
constexpr unsigned OBS_WAIT_LIMIT = 1u << 18;    // try_wait rounds before a wait gives up (a wait normally ends within microseconds)

__device__ __forceinline__ uint32_t obs_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float obs_ex2(float x) {         // 2^x, one instruction (relative error 2^-22)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float OBS_LOG2E = 1.4426950408889634f;

template <bool BF16>
__device__ __forceinline__ float obs_round(float x) {     // to the model's 16-bit type and back
  return BF16 ? __bfloat162float(__float2bfloat16_rn(x)) : __half2float(__float2half_rn(x));
}
template <bool BF16>
__device__ __forceinline__ uint32_t obs_pack(float lo, float hi) {   // two values rounded to the 16-bit type
  if (BF16) { const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&v); }
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <bool BF16>
__device__ __forceinline__ float obs_unpack(uint32_t bits16) {
  return BF16 ? __uint_as_float(bits16 << 16) : h2f((uint16_t)bits16);
}
template <bool BF16>
__device__ __forceinline__ float2 obs_unpack2(uint32_t w) {          // both halves of a packed pair
  if (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <bool BF16>
__device__ __forceinline__ uint32_t obs_max2(uint32_t a, uint32_t b) {   // element-wise maximum of two packed pairs
  if (BF16) {
    const __nv_bfloat162 v = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&v);
}
// A pair of accumulator values as the pair of scores the reference sees: the 16-bit matmul result
// times 1/sqrt(128) in fp32, rounded to the 16-bit type again (two values per conversion).
template <bool BF16>
__device__ __forceinline__ uint32_t obs_score2(uint32_t acc_lo, uint32_t acc_hi) {
  const float2 f = obs_unpack2<BF16>(obs_pack<BF16>(__uint_as_float(acc_lo), __uint_as_float(acc_hi)));
  return obs_pack<BF16>(f.x * INV_SQRT_D, f.y * INV_SQRT_D);
}

// ── mbarrier, TMA, tcgen05 ──────────────────────────────────────────────────────────────────
__device__ __forceinline__ void obs_bar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void obs_bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void obs_bar_arrive_tx(uint32_t bar, uint32_t bytes) {   // arrive and expect `bytes` of copies
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Waits (bounded) for the barrier's phase `parity` to complete; false if it did not.
__device__ __forceinline__ bool obs_bar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned spins = 0; spins < OBS_WAIT_LIMIT; ++spins) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// One box of a 3-D tensor map into shared memory; its bytes are counted on the mbarrier.
__device__ __forceinline__ void obs_tma_3d(uint32_t dst, const CUtensorMap* tm, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
               : "memory");
}
// Shared-memory matrix descriptor of a K-major operand with 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart.  Bits [0,14) start address / 16, [16,30) leading-dimension
// offset / 16 (unused with a swizzle: 1), [32,46) offset between 8-row groups / 16, [46,48)
// descriptor version 1, [61,64) layout 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t obs_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | (uint64_t)1 << 16 | (uint64_t)(1024 >> 4) << 32 | (uint64_t)1 << 46 |
         (uint64_t)2 << 61;
}
// Instruction descriptor of a dense 16-bit MMA of 128 x n (n a multiple of 16) with fp32
// accumulation, both operands K-major: bits [4,6) accumulator 1 = fp32, [7,10) and [10,13) operand
// types (0 = fp16, 1 = bf16), [17,23) N / 8, [24,29) M / 16.
template <bool BF16>
__device__ __forceinline__ constexpr uint32_t obs_idesc(int n) {
  return 1u << 4 | (BF16 ? 1u : 0u) << 7 | (BF16 ? 1u : 0u) << 10 | (uint32_t)(n >> 3) << 17 | (uint32_t)(128 >> 4) << 24;
}
__device__ __forceinline__ void obs_mma(uint32_t tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void obs_commit(uint32_t bar) {   // the barrier gets an arrival once the MMAs issued so far are done
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void obs_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void obs_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 32 consecutive fp32 columns of this thread's accumulator row (lane i of warp w: row 32*(w&3)+i);
// the wait is part of the statement so that no use of the registers can move ahead of it.
__device__ __forceinline__ void obs_tmem_ld(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// Byte offset, inside an operand of `panel` bytes per 64 channels, of 16-byte chunk c16 (8
// channels; 0..15) of row `row`: rows of 128 bytes, the chunk's place within its row XORed with the
// row's place within its group of 8.
__device__ __forceinline__ uint32_t obs_off(int row, int c16, int panel) {
  return (uint32_t)((c16 >> 3) * panel + row * 128 + (((c16 & 7) ^ (row & 7)) << 4));
}

// `rows` rows of 128 16-bit elements (row stride in elements) into operand rows row0.. of the
// operand at dst, by plain loads; rows >= rows_valid are zero-filled.
__device__ __forceinline__ void obs_stage(unsigned char* dst, int panel, int row0, const uint16_t* src, int64_t row_stride,
                                          int rows, int rows_valid, bool aligned) {
  for (int i = threadIdx.x; i < rows * 16; i += OBS_THREADS) {
    const int row = i >> 4, c16 = i & 15;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_valid) {
      const uint16_t* p = src + (int64_t)row * row_stride + c16 * 8;
      if (aligned) v = *reinterpret_cast<const uint4*>(p);
      else {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) w[e] = (uint32_t)p[2 * e] | (uint32_t)p[2 * e + 1] << 16;
        v = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    *reinterpret_cast<uint4*>(dst + obs_off(row0 + row, c16, panel)) = v;
  }
}

struct ObsArgs {
  const uint16_t* q; const uint16_t* k;
  int64_t q_head_stride, q_row_stride, k_head_stride, k_row_stride;   // elements
  int g, W, T, causal, n_tiles;
  int BH, P;           // heads; CTAs per head (CTA x of a head takes tiles x, x+P, ...)
  int extra_rows;      // rows of the second pass's grid that compute channel scores
  int n_pad;           // query rows rounded up to a multiple of 64: N of the second pass's MMAs
  int tma_q, tma_k;    // operands come through the tensor maps (else by plain loads)
  float* part;         // [BH][2*P][R][2] maxima and sums per (CTA, half of a tile's keys)
  float* ksq;          // [BH][P][128] sums of k^2 per CTA
  float* stats;        // [BH][R][2] maxima and sums over all keys
  float* token;        // [BH][T]
  float* channel;      // [BH][128]
  int* status;         // bit 0: operands did not arrive, bit 1: products did not complete
};

// The channel score of KV head bh = mean(q^2) * mean_t(k^2), by one CTA of OBS_THREADS threads:
// threads (half, channel) sum every other row / CTA sum, the halves are added at the end.  Runs as
// an extra CTA of the second pass (the k^2 sums come from the first).
template <bool BF16>
__device__ __forceinline__ void obs_channel_score(const ObsArgs& A, int bh, float* s_sum /* [4][128] */) {
  const int tid = threadIdx.x, c = tid & 127, half = tid >> 7, R = A.g * A.W;
  float qs = 0.f, ks = 0.f;
#pragma unroll 8
  for (int row = half; row < R; row += 2) {
    const uint16_t b = A.q[((int64_t)bh * A.g + row / A.W) * A.q_head_stride + (int64_t)(row % A.W) * A.q_row_stride + c];
    const float x = obs_unpack<BF16>(b);
    qs = fmaf(x, x, qs);
  }
#pragma unroll 16
  for (int i = half; i < A.P; i += 2) ks += A.ksq[((int64_t)bh * A.P + i) * 128 + c];
  s_sum[half * 128 + c] = qs; s_sum[256 + half * 128 + c] = ks;
  __syncthreads();
  if (tid < 128)
    A.channel[(int64_t)bh * 128 + tid] = ((s_sum[tid] + s_sum[128 + tid]) / (float)R) * ((s_sum[256 + tid] + s_sum[384 + tid]) / (float)A.T);
}

// PASS 0: row statistics and k^2 sums.  PASS 1: token scores; the first extra_rows rows of its grid
// (dispatched first) compute the heads' channel scores instead.
template <bool BF16, int PASS>
__global__ void __launch_bounds__(OBS_THREADS, 2)
obs_stream_kernel(const ObsArgs A, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k) {
  extern __shared__ unsigned char obs_raw[];
  __shared__ __align__(8) uint64_t s_bar[4];                 // [b] key buffer b has landed (the first time with the queries), [2+b] products into accumulator b complete
  __shared__ uint32_t s_tmem;                                // base of the CTA's tensor-memory columns
  __shared__ float s_col[4 * OBS_KEYS];                      // PASS 1: the two row halves' sums per key; channel CTAs: their partial sums
  __shared__ __align__(16) float2 s_ci[OBS_MAX_ROWS];        // PASS 1: per query row (M * log2 e, 1 / L); (0, 0) past R
  __shared__ __align__(16) int s_lim[OBS_MAX_ROWS];          // PASS 1: last key the row may see
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (PASS == 1 && (int)blockIdx.y < A.extra_rows) {        // the grid's first rows: one CTA per head for the channel scores
    const int head = blockIdx.y * gridDim.x + blockIdx.x;
    if (head < A.BH) obs_channel_score<BF16>(A, head, s_col);
    return;
  }
  const int cx = blockIdx.x, bh = PASS == 1 ? (int)blockIdx.y - A.extra_rows : (int)blockIdx.y;
  const int R = A.g * A.W, T = A.T, MB = (R + OBS_ROWS - 1) / OBS_ROWS, P = A.P;
  const int n_my = (A.n_tiles - cx + P - 1) / P;             // tiles cx, cx+P, ... (P <= n_tiles: at least one)
  const int q_panel = MB * OBS_PANEL;                        // the queries: [MB*128 rows] x 64 channels, twice
  const uint32_t raw32 = obs_smem(obs_raw), k32 = (raw32 + 1023u) & ~1023u, q32 = k32 + 2 * OBS_BLOCK;
  unsigned char* s_k = obs_raw + (k32 - raw32);              // two key buffers of OBS_BLOCK bytes, 1024-byte aligned
  unsigned char* s_q = s_k + 2 * OBS_BLOCK;
  const uint32_t bar0 = obs_smem(&s_bar[0]);
  // accumulator columns: PASS 0 one column per key and row block, PASS 1 one per (padded) query row; two accumulators
  const uint32_t acc_cols = PASS == 0 ? (uint32_t)MB * OBS_KEYS : (A.n_pad <= 128 ? 128u : 256u);
  const uint32_t tmem_cols = 2 * acc_cols;
  const bool k_al = (A.k_row_stride & 7) == 0 && (A.k_head_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(A.k) & 15) == 0;
  const uint16_t* k_head = A.k + bh * A.k_head_stride;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) obs_bar_init(bar0 + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                                           // this warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(obs_smem(&s_tmem)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // query rows past R are zeros; operands that do not come by TMA are staged here (the first two key tiles)
  for (int i = tid; i < (MB * OBS_ROWS - R) * 16; i += OBS_THREADS)
    *reinterpret_cast<uint4*>(s_q + obs_off(R + (i >> 4), i & 15, q_panel)) = make_uint4(0u, 0u, 0u, 0u);
  if (!A.tma_q) {
    const bool al = (A.q_row_stride & 7) == 0 && (A.q_head_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(A.q) & 15) == 0;
    for (int gi = 0; gi < A.g; ++gi)                         // row gi*W + w = query head gi of the group, window position w
      obs_stage(s_q, q_panel, gi * A.W, A.q + ((int64_t)bh * A.g + gi) * A.q_head_stride, A.q_row_stride, A.W, A.W, al);
  }
  if (!A.tma_k)
    for (int n = 0; n < min(n_my, 2); ++n) {
      const int t0 = (cx + n * P) * OBS_KEYS;
      obs_stage(s_k + n * OBS_BLOCK, OBS_PANEL, 0, k_head + (int64_t)t0 * A.k_row_stride, A.k_row_stride, OBS_KEYS,
                min(OBS_KEYS, T - t0), k_al);
    }
  if (PASS == 1)
    for (int r = tid; r < OBS_MAX_ROWS; r += OBS_THREADS) {
      float2 ci = make_float2(0.f, 0.f);
      if (r < R) {
        const float2 ml = *reinterpret_cast<const float2*>(A.stats + ((int64_t)bh * R + r) * 2);
        ci = make_float2(ml.x * OBS_LOG2E, __frcp_rn(ml.y));
      }
      s_ci[r] = ci;
      s_lim[r] = A.causal ? T - A.W + (r % A.W) : T - 1;
    }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the plain stores above, as the tensor cores will see them
  obs_fence_before();
  __syncthreads();
  obs_fence_after();
  const uint32_t tmem = s_tmem;

  // thread 0: the copies of key tile n into buffer n & 1 (with the queries the first time), or the arrival that stands for them
  auto load_tile = [&](int n, bool with_q) {
    const uint32_t bar = bar0 + 8 * (n & 1);
    const uint32_t tx = (A.tma_k ? (uint32_t)OBS_BLOCK : 0u) + (with_q && A.tma_q ? (uint32_t)R * 256u : 0u);
    if (tx == 0) { obs_bar_arrive(bar); return; }
    obs_bar_arrive_tx(bar, tx);
    if (A.tma_k) {                                           // two boxes of 64 channels (rows past T arrive as zeros)
      const uint32_t dst = k32 + (uint32_t)(n & 1) * OBS_BLOCK;
      const int t0 = (cx + n * P) * OBS_KEYS;
      obs_tma_3d(dst, &tm_k, 0, t0, bh, bar);
      obs_tma_3d(dst + OBS_PANEL, &tm_k, 64, t0, bh, bar);
    }
    if (with_q && A.tma_q)
      for (int gi = 0; gi < A.g; ++gi) {                     // the W rows of query head gi (W is a multiple of 8 here)
        const uint32_t dst = q32 + (uint32_t)(gi * A.W) * 128u;
        obs_tma_3d(dst, &tm_q, 0, 0, bh * A.g + gi, bar);
        obs_tma_3d(dst + (uint32_t)q_panel, &tm_q, 64, 0, bh * A.g + gi, bar);
      }
  };
  // thread 0: once tile n's operands are there, its products into accumulator n & 1
  auto issue_tile = [&](int n) {
    const int b = n & 1;
    if (!obs_bar_wait(bar0 + 8 * b, (uint32_t)(n >> 1) & 1u)) {
      atomicOr(A.status, 1);
      obs_bar_wait(bar0 + 8 * b, (uint32_t)(n >> 1) & 1u);   // (one more bounded wait for the copies in flight)
      obs_bar_arrive(bar0 + 8 * (2 + b));
      return;
    }
    obs_fence_after();
    const uint32_t kb = k32 + (uint32_t)b * OBS_BLOCK, acc = tmem + (uint32_t)b * acc_cols;
    if (PASS == 0) {                                         // S = Q.K^T per 128-row block
      const uint32_t idesc = obs_idesc<BF16>(OBS_KEYS);
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)                       // 16 channels a step: 32 bytes along the swizzled row, the second panel after four
          obs_mma(acc + (uint32_t)mb * OBS_KEYS,
                  obs_desc(q32 + (uint32_t)(kk >> 2) * q_panel + (uint32_t)mb * OBS_PANEL + (uint32_t)(kk & 3) * 32u),
                  obs_desc(kb + (uint32_t)(kk >> 2) * OBS_PANEL + (uint32_t)(kk & 3) * 32u), idesc, kk > 0 ? 1u : 0u);
    } else {                                                 // S^T = K.Q^T: all (padded) query rows at once
      const uint32_t idesc = obs_idesc<BF16>(A.n_pad);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        obs_mma(acc, obs_desc(kb + (uint32_t)(kk >> 2) * OBS_PANEL + (uint32_t)(kk & 3) * 32u),
                obs_desc(q32 + (uint32_t)(kk >> 2) * q_panel + (uint32_t)(kk & 3) * 32u), idesc, kk > 0 ? 1u : 0u);
    }
    obs_commit(bar0 + 8 * (2 + b));
  };

  if (tid == 0) {
    load_tile(0, true);
    if (n_my > 1) load_tile(1, false);
    issue_tile(0);
  }

  const int q4 = warp & 3, half = warp >> 2;
  // PASS 0: a thread's rows (one per row block), their running statistics over this half of the keys; its share of k^2
  float run_m[2] = {-INFINITY, -INFINITY}, run_l[2] = {0.f, 0.f};
  float ksq_acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int c16 = warp * 2 + (lane >> 4), rs = lane & 15;    // k^2: this thread's 16-byte chunk and set of keys

#pragma unroll 1
  for (int n = 0; n < n_my; ++n) {
    const int b = n & 1, tile = cx + n * P, t0 = tile * OBS_KEYS, n_keys = min(OBS_KEYS, T - t0);
    if (tid == 0 && !obs_bar_wait(bar0 + 8 * (2 + b), (uint32_t)(n >> 1) & 1u)) atomicOr(A.status, 2);
    __syncthreads();                                         // tile n's products are complete (and everybody is done with tile n-1)
    obs_fence_after();
    if (tid == 0) {
      // PASS 1 reads no keys from shared memory: buffer b is free now that tile n's products are done,
      // and tile n+2 gets the whole of this tile's work to arrive
      if (PASS == 1 && A.tma_k && n + 2 < n_my) load_tile(n + 2, false);
      if (n + 1 < n_my) issue_tile(n + 1);                   // the other accumulator: its last readers passed the barrier above
    }
    // (only tiles that reach into the window or past the sequence's end have anything to mask)
    const bool edge = t0 + OBS_KEYS > (A.causal ? T - A.W : T);
    const uint32_t acc = tmem + (uint32_t)b * acc_cols + ((uint32_t)(q4 * 32) << 16);

    if (PASS == 0) {
      {
        // k^2 of the tile.  Lanes 0-15 / 16-31 of warp w take the 16-byte chunk (8 channels) 2w / 2w+1 of
        // keys rs, rs+16, ...; a quarter warp's loads fall on distinct banks.  (Rows past T are zeros.)
        const unsigned char* src = s_k + b * OBS_BLOCK + obs_off(rs, c16, OBS_PANEL);
#pragma unroll
        for (int j = 0; j < OBS_KEYS / 16; ++j) {            // key j*16 + rs: two groups of 8 rows further each time
          const uint4 v = *reinterpret_cast<const uint4*>(src + j * 2048);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = obs_unpack2<BF16>(w[e]);
            ksq_acc[2 * e] = fmaf(x.x, x.x, ksq_acc[2 * e]); ksq_acc[2 * e + 1] = fmaf(x.y, x.y, ksq_acc[2 * e + 1]);
          }
        }
      }
      if (A.tma_k && n + 2 < n_my) {                         // the k^2 sums were the last readers of buffer b: tile n+2 may come
        __syncthreads();
        if (tid == 0) load_tile(n + 2, false);
      }
      auto stats = [&](auto edge_c) {                        // compiled once with and once without the masking
        constexpr bool EDGE = decltype(edge_c)::value;
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {
          const int row = mb * OBS_ROWS + q4 * 32 + lane;
          if (mb >= MB || row - lane >= R) continue;         // (the whole warp)
          const int lim = A.causal ? T - A.W + (row % A.W) : T - 1;   // last key this row may see
          const int tk = t0 + half * 64;
          float m = run_m[mb], l = run_l[mb];
          // 32 keys at a time: the scores (as packed pairs), the row's maximum over them, one exponential each
#pragma unroll 1
          for (int ck = 0; ck < 2; ++ck) {
            uint32_t v[32];
            obs_tmem_ld(acc + (uint32_t)(mb * OBS_KEYS + half * 64 + ck * 32), v);
            uint32_t h2 = BF16 ? 0xFF80FF80u : 0xFC00FC00u;  // (-inf, -inf)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              uint32_t s2 = obs_score2<BF16>(v[2 * i], v[2 * i + 1]);
              if (EDGE) {
                const int t = tk + ck * 32 + 2 * i;
                if (t > lim) s2 = (s2 & 0xFFFF0000u) | (BF16 ? 0xFF80u : 0xFC00u);
                if (t + 1 > lim) s2 = (s2 & 0x0000FFFFu) | (BF16 ? 0xFF800000u : 0xFC000000u);
              }
              v[i] = s2;
              h2 = obs_max2<BF16>(h2, s2);
            }
            const float2 hh = obs_unpack2<BF16>(h2);
            const float nm = fmaxf(m, fmaxf(hh.x, hh.y));
            const float c = nm > -INFINITY ? nm * OBS_LOG2E : 0.f;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 16; ++i) {                   // (2^-inf = 0: masked keys add nothing)
              const float2 sc = obs_unpack2<BF16>(v[i]);
              sum[(2 * i) & 3] += obs_ex2(fmaf(sc.x, OBS_LOG2E, -c));
              sum[(2 * i + 1) & 3] += obs_ex2(fmaf(sc.y, OBS_LOG2E, -c));
            }
            l = (m > -INFINITY ? l * obs_ex2(fmaf(m, OBS_LOG2E, -c)) : 0.f) + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
            m = nm;
          }
          run_m[mb] = m; run_l[mb] = l;
        }
      };
      if (edge) stats(std::true_type{});
      else stats(std::false_type{});
    } else {
      // this thread's key against its half of the (padded) query rows, 32 at a time; the weights are
      // rounded to the 16-bit type as the reference's softmax output is and summed inside the thread
      const int t = t0 + q4 * 32 + lane, rows_half = A.n_pad >> 1;
      float colsum = 0.f;
      auto sums = [&](auto edge_c) {
        constexpr bool EDGE = decltype(edge_c)::value;
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int r0 = half * rows_half; r0 < (half + 1) * rows_half; r0 += 32) {
          uint32_t v[32];
          obs_tmem_ld(acc + (uint32_t)r0, v);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float2 sc = obs_unpack2<BF16>(obs_score2<BF16>(v[i], v[i + 1]));
            const float4 ci = *reinterpret_cast<const float4*>(&s_ci[r0 + i]);   // (all lanes the same address)
            if (EDGE) {
              const int2 lim = *reinterpret_cast<const int2*>(&s_lim[r0 + i]);
              if (t > lim.x) sc.x = -INFINITY;
              if (t > lim.y) sc.y = -INFINITY;
            }
            const float2 p = obs_unpack2<BF16>(obs_pack<BF16>(obs_ex2(fmaf(sc.x, OBS_LOG2E, -ci.x)) * ci.y,
                                                              obs_ex2(fmaf(sc.y, OBS_LOG2E, -ci.z)) * ci.w));
            a[(i >> 1) & 3] += p.x + p.y;
          }
        }
        colsum = (a[0] + a[1]) + (a[2] + a[3]);
      };
      if (edge) sums(std::true_type{});
      else sums(std::false_type{});
      s_col[half * OBS_KEYS + q4 * 32 + lane] = colsum;
    }
    obs_fence_before();
    __syncthreads();                                         // everybody is done with key buffer b and accumulator b
    if (!A.tma_k && n + 2 < n_my) {                          // without TMA: tile n+2 into the buffer by plain loads, here
      const int t2 = (cx + (n + 2) * P) * OBS_KEYS;
      obs_stage(s_k + b * OBS_BLOCK, OBS_PANEL, 0, k_head + (int64_t)t2 * A.k_row_stride, A.k_row_stride, OBS_KEYS,
                min(OBS_KEYS, T - t2), k_al);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (tid == 0) load_tile(n + 2, false);                 // (the arrival that stands for the copies; the products are issued after the next CTA barrier)
    }
    if (PASS == 1 && tid < n_keys)                           // (the reference's aw.sum(...) is in aw's type)
      A.token[(int64_t)bh * T + t0 + tid] = obs_round<BF16>(s_col[tid] + s_col[OBS_KEYS + tid]);
  }

  if (PASS == 0) {
#pragma unroll
    for (int mb = 0; mb < 2; ++mb) {
      const int row = mb * OBS_ROWS + q4 * 32 + lane;
      if (mb < MB && row < R)
        *reinterpret_cast<float2*>(A.part + ((((int64_t)bh * P + cx) * 2 + half) * R + row) * 2) = make_float2(run_m[mb], run_l[mb]);
    }
    // the 16 lanes of a chunk add their k^2 up along a fixed tree
#pragma unroll
    for (int o = 1; o < 16; o <<= 1)
#pragma unroll
      for (int e = 0; e < 8; ++e) ksq_acc[e] += __shfl_xor_sync(0xffffffffu, ksq_acc[e], o);
    if (rs == 0) {
      float4* dst = reinterpret_cast<float4*>(A.ksq + ((int64_t)bh * P + cx) * 128 + c16 * 8);
      dst[0] = make_float4(ksq_acc[0], ksq_acc[1], ksq_acc[2], ksq_acc[3]);
      dst[1] = make_float4(ksq_acc[4], ksq_acc[5], ksq_acc[6], ksq_acc[7]);
    }
  }
  // (the loop's last barrier came after every read of tensor memory)
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// The rows' maxima and sums over the first pass's CTAs.  A CTA takes 8 rows of a head: thread (slice, row)
// merges every 64th partial result of its row (a warp's loads cover 4 slices x 8 rows = 4 runs of 64
// bytes), the 64 slices of a row are then merged by one warp along a fixed tree.
constexpr int OBS_RED_ROWS = 8;
constexpr int OBS_RED_SLICES = 64;
constexpr int OBS_RED_THREADS = OBS_RED_ROWS * OBS_RED_SLICES;
__device__ __forceinline__ void obs_merge(float& M, float& L, float m, float l) {   // (M, L) <- (M, L) + (m, l)
  if (m > -INFINITY) {
    const float n = fmaxf(M, m);
    L = L * obs_ex2((M - n) * OBS_LOG2E) + l * obs_ex2((m - n) * OBS_LOG2E);
    M = n;
  }
}
__global__ void __launch_bounds__(OBS_RED_THREADS)
obs_reduce_kernel(ObsArgs A) {
  __shared__ float2 s_ml[OBS_RED_SLICES][OBS_RED_ROWS];
  const int bh = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int R = A.g * A.W, n_parts = 2 * A.P;
  const int r = tid & (OBS_RED_ROWS - 1), slice = tid / OBS_RED_ROWS;
  const int row = blockIdx.x * OBS_RED_ROWS + r;
  float M = -INFINITY, L = 0.f;
  if (row < R) {
    const float* p = A.part + ((int64_t)bh * n_parts * R + row) * 2;
    for (int base = slice; base < n_parts; base += 8 * OBS_RED_SLICES) {
      float2 ml[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {                          // eight loads in flight
        const int i = base + u * OBS_RED_SLICES;
        ml[u] = i < n_parts ? *reinterpret_cast<const float2*>(p + (int64_t)i * R * 2) : make_float2(-INFINITY, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) obs_merge(M, L, ml[u].x, ml[u].y);
    }
  }
  s_ml[slice][r] = make_float2(M, L);
  __syncthreads();
  if (warp < OBS_RED_ROWS) {                                 // warp w: the 64 slices of row w
    const float2 a = s_ml[lane][warp], b = s_ml[lane + 32][warp];
    M = a.x; L = a.x > -INFINITY ? a.y : 0.f;
    obs_merge(M, L, b.x, b.y);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, M, o), ol = __shfl_xor_sync(0xffffffffu, L, o);
      const float n = fmaxf(M, om);
      L = n > -INFINITY ? L * obs_ex2((M - n) * OBS_LOG2E) + ol * obs_ex2((om - n) * OBS_LOG2E) : 0.f;
      M = n;
    }
    const int out_row = blockIdx.x * OBS_RED_ROWS + warp;
    if (lane == 0 && out_row < R) *reinterpret_cast<float2*>(A.stats + ((int64_t)bh * R + out_row) * 2) = make_float2(M, L);
  }
}

// ── tensor maps ─────────────────────────────────────────────────────────────────────────────
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, found through the runtime (the library does not link the driver).
static EncodeTiledFn encode_tiled() {
  static const EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return (EncodeTiledFn) nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// A map over [heads][rows][128] 16-bit elements (strides in elements) whose boxes are `box_rows`
// rows of 64 channels, laid down with the 128-byte swizzle; false if the layout cannot be mapped
// (unaligned base or strides, or the encoder is missing), in which case the kernel stages by loads.
static bool obs_map(CUtensorMap* tm, const void* base, bool bf16, int64_t head_stride, int64_t row_stride, int64_t heads,
                    int64_t rows, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr || box_rows < 1 || box_rows > 256) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride & 7) != 0 || (head_stride & 7) != 0) return false;
  if (row_stride < 128 || head_stride <= 0) return false;
  const cuuint64_t dims[3] = {128u, (cuuint64_t)rows, (cuuint64_t)heads};
  const cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2u, (cuuint64_t)head_stride * 2u};
  const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
  const cuuint32_t elem[3] = {1u, 1u, 1u};
  const CUresult r = enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
                         dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int64_t rdkv_obs_scratch_words(int BH, int g, int W, int T) {
  if (BH < 0 || g <= 0 || W <= 0 || T <= 0) return 0;
  const int64_t n_tiles = (T + OBS_KEYS - 1) / OBS_KEYS, R = (int64_t)g * W;   // (sized for one CTA per tile; fewer run)
  return BH * (2 * n_tiles * R * 2 + n_tiles * 128 + R * 2) + 1;
}

extern "C" int rdkv_obs_scores(const void* q_obs, const void* k, int dtype, int64_t q_head_stride,
                               int64_t q_row_stride, int64_t k_head_stride, int64_t k_row_stride, int BH, int g,
                               int W, int T, int causal, float* scratch, float* layer_token, float* layer_channel,
                               void* stream) {
  if (q_obs == nullptr || k == nullptr || scratch == nullptr || layer_token == nullptr || layer_channel == nullptr)
    return RDKV_ERR_BAD_ARG;
  if (dtype != RDKV_F16 && dtype != RDKV_BF16) return RDKV_ERR_BAD_ARG;
  if (BH < 0 || g <= 0 || W <= 0 || T <= 0 || (causal && W > T)) return RDKV_ERR_BAD_SHAPE;
  if ((int64_t)g * W > OBS_MAX_ROWS) return RDKV_ERR_TOO_LARGE;
  if (BH == 0) return RDKV_OK;
  if (BH > 65000) return RDKV_ERR_TOO_LARGE;
  const bool bf = dtype == RDKV_BF16;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || sms <= 0) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  ObsArgs A;
  A.q = reinterpret_cast<const uint16_t*>(q_obs); A.k = reinterpret_cast<const uint16_t*>(k);
  A.q_head_stride = q_head_stride; A.q_row_stride = q_row_stride; A.k_head_stride = k_head_stride; A.k_row_stride = k_row_stride;
  A.g = g; A.W = W; A.T = T; A.causal = causal ? 1 : 0; A.n_tiles = (T + OBS_KEYS - 1) / OBS_KEYS;
  const int64_t R = (int64_t)g * W;
  const int MB = (int)((R + OBS_ROWS - 1) / OBS_ROWS);
  // CTAs per head: the resident CTAs (two per SM with one row block, one with two) shared out over the heads
  const int slots = sms * (MB == 1 ? 2 : 1);
  A.BH = BH; A.P = std::min(A.n_tiles, std::max(1, slots / BH));
  A.extra_rows = (BH + A.P - 1) / A.P;
  A.n_pad = (int)((R + 63) / 64) * 64;
  A.part = scratch;
  A.ksq = A.part + (int64_t)BH * 2 * A.n_tiles * R * 2;
  A.stats = A.ksq + (int64_t)BH * A.n_tiles * 128;
  A.status = reinterpret_cast<int*>(A.stats + (int64_t)BH * R * 2);
  A.token = layer_token; A.channel = layer_channel;
  // the operands come by TMA when their layout can be mapped; a head's W query rows are one box,
  // which must start on a group of 8 rows
  CUtensorMap tm_q, tm_k;
  memset(&tm_q, 0, sizeof(tm_q)); memset(&tm_k, 0, sizeof(tm_k));
  A.tma_k = obs_map(&tm_k, k, bf, k_head_stride, k_row_stride, BH, T, OBS_KEYS) ? 1 : 0;
  A.tma_q = (W % 8 == 0 && obs_map(&tm_q, q_obs, bf, q_head_stride, q_row_stride, (int64_t)BH * g, W, W)) ? 1 : 0;
  const size_t smem = 1024 + (size_t)(2 + MB) * OBS_BLOCK;   // (the base is rounded up to 1024 bytes in the kernel)
  cudaStream_t st = (cudaStream_t)stream;
  e = cudaMemsetAsync(A.status, 0, sizeof(int), st);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  auto launch = [&](auto kern_stats, auto kern_token) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern_stats, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern_token, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
    kern_stats<<<dim3(A.P, BH), OBS_THREADS, smem, st>>>(A, tm_q, tm_k);
    int rc = launch_status();
    if (rc != RDKV_OK) return rc;
    obs_reduce_kernel<<<dim3((unsigned)((R + OBS_RED_ROWS - 1) / OBS_RED_ROWS), BH), OBS_RED_THREADS, 0, st>>>(A);
    rc = launch_status();
    if (rc != RDKV_OK) return rc;
    kern_token<<<dim3(A.P, BH + A.extra_rows), OBS_THREADS, smem, st>>>(A, tm_q, tm_k);
    return launch_status();
  };
  if (bf) return launch(obs_stream_kernel<true, 0>, obs_stream_kernel<true, 1>);
  return launch(obs_stream_kernel<false, 0>, obs_stream_kernel<false, 1>);
}
