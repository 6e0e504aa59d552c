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
// The contraction runs on the fifth-generation tensor cores.  Per (KV head, 128-key tile) one CTA
//   * brings the tile's keys and the head's g*W query rows into shared memory in the tensor
//     cores' K-major layout with 128-byte swizzle: tiled TMA copies through two tensor maps when
//     the strides allow it, plain 16-byte loads with the same swizzle otherwise;
//   * has one thread issue eight tcgen05.mma (M = 128 rows, N = 128 keys, K = 16 channels each) per
//     128-row block into an fp32 accumulator in tensor memory, followed by a tcgen05.commit onto
//     an mbarrier;
//   * reads the accumulator back with tcgen05.ld: a thread holds 32 consecutive keys of ONE row at
//     a time, so the row statistics need no exchange between threads.
// Three launches per layer:
//   obs_tile_kernel<.,0>  per tile: scores rounded as the reference's 16-bit matmul and scaling
//                         round them, masked; per row and half tile the maximum and the sum of
//                         exponentials; per channel the tile's sum of k^2.
//   obs_reduce_kernel     per KV head: the rows' maxima and sums over all tiles.
//   obs_tile_kernel<.,1>  per tile: the same scores again, p = exp(s - M) / L rounded to the 16-bit
//                         type, parked in shared memory (over the spent operands) and summed over
//                         the rows: the token scores of the tile.  One more CTA per head turns the
//                         tiles' k^2 sums and the queries into the channel score meanwhile.
// The keys are read twice (the second time mostly from L2); sums run in a fixed order.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets a bit in the status word (the
// last word of the scratch buffer: 1 = the operands did not arrive, 2 = the products did not
// complete), the kernel still frees its tensor memory and returns, and the results are invalid.
#include <cuda.h>   // CUtensorMap and its enums (the encoder itself is looked up through the runtime)

#include <cstring>
#include <type_traits>

#include "rdkv_common.cuh"

namespace rdkv {

constexpr int OBS_THREADS = 256;                 // 8 warps: warp w reads accumulator rows 32*(w&3).., key half w>>2
constexpr int OBS_KEYS = 128;                    // keys per tile = N of one MMA
constexpr int OBS_ROWS = 128;                    // rows per accumulator block = M of one MMA
constexpr int OBS_MAX_ROWS = 256;                // (query head, position) pairs per KV head: two blocks
constexpr int OBS_PANEL = 128 * 128;             // bytes: 128 rows of 64 16-bit channels, 128 bytes a row
constexpr int OBS_BLOCK = 2 * OBS_PANEL;         // a 128-row operand: channels 0-63, then channels 64-127
constexpr int OBS_P_LD = 65;                     // words per row of the parked weights (odd: rows fall on distinct banks)
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
// Instruction descriptor of a dense 16-bit MMA with fp32 accumulation, both operands K-major:
// bits [4,6) accumulator 1 = fp32, [7,10) and [10,13) operand types (0 = fp16, 1 = bf16),
// [17,23) N / 8, [24,29) M / 16.
template <bool BF16>
__device__ __forceinline__ constexpr uint32_t obs_idesc() {
  return 1u << 4 | (BF16 ? 1u : 0u) << 7 | (BF16 ? 1u : 0u) << 10 | (uint32_t)(OBS_KEYS >> 3) << 17 |
         (uint32_t)(OBS_ROWS >> 4) << 24;
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

// Byte offset, inside a 128-row operand, of 16-byte chunk c16 (8 channels; 0..15) of row `row`:
// the chunk's place within its 128-byte row is XORed with the row's place within its group of 8.
__device__ __forceinline__ uint32_t obs_off(int row, int c16) {
  return (uint32_t)((c16 >> 3) * OBS_PANEL + (row >> 3) * 1024 + (row & 7) * 128 + (((c16 & 7) ^ (row & 7)) << 4));
}

// `rows` rows of 128 16-bit elements (row stride in elements) into operand rows row0.. of the
// operand blocks at dst, by plain loads; rows >= rows_valid are zero-filled.
__device__ __forceinline__ void obs_stage(unsigned char* dst, int row0, const uint16_t* src, int64_t row_stride, int rows,
                                          int rows_valid, bool aligned) {
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
    const int r = row0 + row;
    *reinterpret_cast<uint4*>(dst + (size_t)(r >> 7) * OBS_BLOCK + obs_off(r & 127, c16)) = v;
  }
}

struct ObsArgs {
  const uint16_t* q; const uint16_t* k;
  int64_t q_head_stride, q_row_stride, k_head_stride, k_row_stride;   // elements
  int g, W, T, causal, n_tiles;
  int BH, extra_rows;  // heads; rows of the second tile launch's grid that compute channel scores
  int tma_q, tma_k;    // operands come through the tensor maps (else by plain loads)
  float* part;         // [BH][2*n_tiles][R][2] half-tile maxima and sums
  float* ksq;          // [BH][n_tiles][128] tile sums of k^2
  float* stats;        // [BH][R][2] maxima and sums over all keys
  float* token;        // [BH][T]
  float* channel;      // [BH][128]
  int* status;         // bit 0: operands did not arrive, bit 1: products did not complete
};

// The channel score of KV head bh = mean(q^2) * mean_t(k^2), by one CTA of OBS_THREADS threads:
// threads (half, channel) sum every other row / tile, the halves are added at the end.  Runs as an
// extra CTA of the second tile launch (the tiles' k^2 sums come from the first).
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
  for (int i = half; i < A.n_tiles; i += 2) ks += A.ksq[((int64_t)bh * A.n_tiles + i) * 128 + c];
  s_sum[half * 128 + c] = qs; s_sum[256 + half * 128 + c] = ks;
  __syncthreads();
  if (tid < 128)
    A.channel[(int64_t)bh * 128 + tid] = ((s_sum[tid] + s_sum[128 + tid]) / (float)R) * ((s_sum[256 + tid] + s_sum[384 + tid]) / (float)A.T);
}

// PASS 0: row statistics and k^2 sums of a tile.  PASS 1: token scores of a tile; the first
// extra_rows rows of its grid (dispatched first) compute the heads' channel scores instead.
template <bool BF16, int PASS>
__global__ void __launch_bounds__(OBS_THREADS, 3)
obs_tile_kernel(const ObsArgs A, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k) {
  extern __shared__ unsigned char obs_raw[];
  __shared__ __align__(8) uint64_t s_bar[2];                 // [0] operands landed, [1] products complete
  __shared__ uint32_t s_tmem;                                // base of the CTA's tensor-memory columns
  __shared__ float s_col[4 * OBS_KEYS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (PASS == 1 && (int)blockIdx.y < A.extra_rows) {        // the grid's first rows: one CTA per head for the channel scores
    const int head = blockIdx.y * gridDim.x + blockIdx.x;
    if (head < A.BH) obs_channel_score<BF16>(A, head, s_col);
    return;
  }
  const int tile = blockIdx.x, bh = PASS == 1 ? (int)blockIdx.y - A.extra_rows : (int)blockIdx.y;
  const int R = A.g * A.W, T = A.T, MB = (R + OBS_ROWS - 1) / OBS_ROWS;
  const uint32_t raw32 = obs_smem(obs_raw), k32 = (raw32 + 1023u) & ~1023u, q32 = k32 + OBS_BLOCK;
  unsigned char* s_k = obs_raw + (k32 - raw32);              // [128 keys] operand block, 1024-byte aligned
  unsigned char* s_q = s_k + OBS_BLOCK;                      // [MB] operand blocks of query rows
  const uint32_t bar_ld = obs_smem(&s_bar[0]), bar_mma = obs_smem(&s_bar[1]);
  const int t0 = tile * OBS_KEYS, n_keys = min(OBS_KEYS, T - t0);
  const uint32_t tmem_cols = MB == 1 ? 128u : 256u;          // one fp32 column per key and row block

  if (tid == 0) {
    obs_bar_init(bar_ld, 1); obs_bar_init(bar_mma, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                                           // this warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(obs_smem(&s_tmem)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // rows past R of the last block are zeros; operands that do not come by TMA are staged here
  for (int i = tid; i < (MB * OBS_ROWS - R) * 16; i += OBS_THREADS) {
    const int r = R + (i >> 4);
    *reinterpret_cast<uint4*>(s_q + (size_t)(r >> 7) * OBS_BLOCK + obs_off(r & 127, i & 15)) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (!A.tma_k) {
    const bool al = (A.k_row_stride & 7) == 0 && (A.k_head_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(A.k) & 15) == 0;
    obs_stage(s_k, 0, A.k + bh * A.k_head_stride + (int64_t)t0 * A.k_row_stride, A.k_row_stride, OBS_KEYS, n_keys, al);
  }
  if (!A.tma_q) {
    const bool al = (A.q_row_stride & 7) == 0 && (A.q_head_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(A.q) & 15) == 0;
    for (int gi = 0; gi < A.g; ++gi)                         // row gi*W + w = query head gi of the group, window position w
      obs_stage(s_q, gi * A.W, A.q + ((int64_t)bh * A.g + gi) * A.q_head_stride, A.q_row_stride, A.W, A.W, al);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the plain stores above, as the tensor cores will see them
  obs_fence_before();
  __syncthreads();
  obs_fence_after();
  const uint32_t tmem = s_tmem;

  if (tid == 0) {
    const uint32_t tx = (A.tma_k ? (uint32_t)OBS_BLOCK : 0u) + (A.tma_q ? (uint32_t)R * 256u : 0u);
    if (tx != 0) {
      obs_bar_arrive_tx(bar_ld, tx);
      if (A.tma_k) {                                         // keys t0.. of head bh: two boxes of 64 channels (rows past T arrive as zeros)
        obs_tma_3d(k32, &tm_k, 0, t0, bh, bar_ld);
        obs_tma_3d(k32 + OBS_PANEL, &tm_k, 64, t0, bh, bar_ld);
      }
      if (A.tma_q)
        for (int gi = 0; gi < A.g; ++gi) {                   // the W rows of query head gi (W is a multiple of 8 here and no box straddles two blocks)
          const int r0 = gi * A.W;
          const uint32_t dst = q32 + (uint32_t)(r0 >> 7) * OBS_BLOCK + (uint32_t)(r0 & 127) * 128u;
          obs_tma_3d(dst, &tm_q, 0, 0, bh * A.g + gi, bar_ld);
          obs_tma_3d(dst + OBS_PANEL, &tm_q, 64, 0, bh * A.g + gi, bar_ld);
        }
    } else {
      obs_bar_arrive(bar_ld);
    }
    if (obs_bar_wait(bar_ld, 0)) {
      obs_fence_after();
      constexpr uint32_t idesc = obs_idesc<BF16>();
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {                     // 16 channels a step: 32 bytes along the swizzled row, the second panel after four
          const uint32_t o = (uint32_t)(kk >> 2) * OBS_PANEL + (uint32_t)(kk & 3) * 32u;
          obs_mma(tmem + (uint32_t)mb * OBS_KEYS, obs_desc(q32 + (uint32_t)mb * OBS_BLOCK + o), obs_desc(k32 + o), idesc,
                  kk > 0 ? 1u : 0u);
        }
      obs_commit(bar_mma);
    } else {                                                 // give the copies one more bounded wait, then let the others go on
      atomicOr(A.status, 1);
      obs_bar_wait(bar_ld, 0);
      obs_bar_arrive(bar_mma);
    }
  }

  if (PASS == 0) {
    // k^2 of the tile.  Lanes 0-15 / 16-31 of warp w take the 16-byte chunk (8 channels) 2w / 2w+1 of
    // keys rs, rs+16, ... (rs = lane & 15); a quarter warp's loads fall on distinct banks.  The 16
    // lanes of a chunk then add up along a fixed tree.  (Rows past the tile's keys are zeros.)
    obs_bar_wait(bar_ld, 0);
    const int c16 = warp * 2 + (lane >> 4), rs = lane & 15;
    const unsigned char* src = s_k + (c16 >> 3) * OBS_PANEL + (rs >> 3) * 1024 + (rs & 7) * 128 + (((c16 & 7) ^ (rs & 7)) << 4);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < OBS_KEYS / 16; ++j) {                // key j*16 + rs: two groups of 8 rows further each time
      const uint4 v = *reinterpret_cast<const uint4*>(src + j * 2048);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = obs_unpack2<BF16>(w[e]);
        acc[2 * e] = fmaf(x.x, x.x, acc[2 * e]); acc[2 * e + 1] = fmaf(x.y, x.y, acc[2 * e + 1]);
      }
    }
#pragma unroll
    for (int o = 1; o < 16; o <<= 1)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
    if (rs == 0) {
      float4* dst = reinterpret_cast<float4*>(A.ksq + ((int64_t)bh * A.n_tiles + tile) * 128 + c16 * 8);
      dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]); dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }

  if (!obs_bar_wait(bar_mma, 0) && lane == 0) atomicOr(A.status, 2);
  __syncwarp();
  obs_fence_after();
  const int q4 = warp & 3, half = warp >> 2;
  // (only tiles that reach into the window or past the sequence's end have anything to mask)
  const bool edge = t0 + OBS_KEYS > (A.causal ? T - A.W : T);
  uint32_t* s_p = reinterpret_cast<uint32_t*>(s_k);          // PASS 1: [R][OBS_P_LD] pairs of weights, over the spent operands
  // the tile's epilogue, compiled once with and once without the masking
  auto epilogue = [&](auto edge_c) {
    constexpr bool EDGE = decltype(edge_c)::value;
    for (int mb = 0; mb < MB; ++mb) {
      const int row = mb * OBS_ROWS + q4 * 32 + lane;
      if (row - lane >= R) continue;                           // (the whole warp)
      const int lim = A.causal ? T - A.W + (row % A.W) : T - 1;   // last key this row may see
      const uint32_t taddr = tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(mb * OBS_KEYS + half * 64);
      const int tk = t0 + half * 64;
      if (PASS == 0) {
        // 32 keys at a time: the scores (as packed pairs), the row's maximum over them, one exponential
        // each; the chunks merge like tiles
        float m = -INFINITY, l = 0.f;
  #pragma unroll 1
        for (int ck = 0; ck < 2; ++ck) {
          uint32_t v[32];
          obs_tmem_ld(taddr + (uint32_t)ck * 32u, v);
          uint32_t h2 = BF16 ? 0xFF80FF80u : 0xFC00FC00u;      // (-inf, -inf)
  #pragma unroll
          for (int i = 0; i < 16; ++i) {
            uint32_t s2 = obs_score2<BF16>(v[2 * i], v[2 * i + 1]);
            if (EDGE) {                                        // (per CTA: only the last tiles mask anything)
              const int t = tk + ck * 32 + 2 * i;
              if (t > lim) s2 = (s2 & 0xFFFF0000u) | (BF16 ? 0xFF80u : 0xFC00u);
              if (t + 1 > lim) s2 = (s2 & 0x0000FFFFu) | (BF16 ? 0xFF800000u : 0xFC000000u);
            }
            v[i] = s2;
            h2 = obs_max2<BF16>(h2, s2);
          }
          const float2 hh = obs_unpack2<BF16>(h2);
          const float n = fmaxf(m, fmaxf(hh.x, hh.y));
          const float c = n > -INFINITY ? n * OBS_LOG2E : 0.f;
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
  #pragma unroll
          for (int i = 0; i < 16; ++i) {                       // (2^-inf = 0: masked keys add nothing)
            const float2 sc = obs_unpack2<BF16>(v[i]);
            sum[(2 * i) & 3] += obs_ex2(fmaf(sc.x, OBS_LOG2E, -c));
            sum[(2 * i + 1) & 3] += obs_ex2(fmaf(sc.y, OBS_LOG2E, -c));
          }
          l = (m > -INFINITY ? l * obs_ex2(fmaf(m, OBS_LOG2E, -c)) : 0.f) + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
          m = n;
        }
        if (row < R)
          *reinterpret_cast<float2*>(A.part + ((((int64_t)bh * A.n_tiles + tile) * 2 + half) * R + row) * 2) = make_float2(m, l);
      } else {
        const float* st = A.stats + ((int64_t)bh * R + min(row, R - 1)) * 2;
        const float cM = st[0] * OBS_LOG2E, inv = __frcp_rn(st[1]);
        uint32_t* prow = s_p + (size_t)min(row, R - 1) * OBS_P_LD + half * 32;
  #pragma unroll 1
        for (int ck = 0; ck < 2; ++ck) {
          uint32_t v[32];
          obs_tmem_ld(taddr + (uint32_t)ck * 32u, v);
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float2 sc = obs_unpack2<BF16>(obs_score2<BF16>(v[i], v[i + 1]));
            if (EDGE) {
              if (tk + ck * 32 + i > lim) sc.x = -INFINITY;
              if (tk + ck * 32 + i + 1 > lim) sc.y = -INFINITY;
            }
            // p = exp(s - M) / L in fp32, rounded to the 16-bit type as the reference's softmax output is
            const uint32_t pp = obs_pack<BF16>(obs_ex2(fmaf(sc.x, OBS_LOG2E, -cM)) * inv, obs_ex2(fmaf(sc.y, OBS_LOG2E, -cM)) * inv);
            if (row < R) prow[ck * 16 + (i >> 1)] = pp;
          }
        }
      }
    }
  };
  if (edge) epilogue(std::true_type{});
  else epilogue(std::false_type{});
  obs_fence_before();
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
  if (PASS == 1) {
    // column sums: thread = (quarter of the rows, pair of keys), rows in order; then the quarters in order
    const int cp = tid & 63, qtr = tid >> 6, per = MB * 32;
    const int r_end = min(R, (qtr + 1) * per);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
    for (int r = qtr * per; r < r_end; ++r) {
      const uint32_t w = s_p[(size_t)r * OBS_P_LD + cp];
      const float2 p = obs_unpack2<BF16>(w);
      a0 += p.x; a1 += p.y;
    }
    s_col[qtr * OBS_KEYS + 2 * cp] = a0; s_col[qtr * OBS_KEYS + 2 * cp + 1] = a1;
    __syncthreads();
    if (tid < n_keys) {
      const float v = ((s_col[tid] + s_col[OBS_KEYS + tid]) + s_col[2 * OBS_KEYS + tid]) + s_col[3 * OBS_KEYS + tid];
      A.token[(int64_t)bh * T + t0 + tid] = obs_round<BF16>(v);      // (the reference's aw.sum(...) is in aw's type)
    }
  }
}

// The rows' maxima and sums over all half tiles.  A CTA takes 8 rows of a head: thread (slice, row)
// merges every 64th half tile of its row (a warp's loads cover 4 slices x 8 rows = 4 runs of 64
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
  const int R = A.g * A.W, n_parts = 2 * A.n_tiles;
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
  const int64_t n_tiles = (T + OBS_KEYS - 1) / OBS_KEYS, R = (int64_t)g * W;
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
  ObsArgs A;
  A.q = reinterpret_cast<const uint16_t*>(q_obs); A.k = reinterpret_cast<const uint16_t*>(k);
  A.q_head_stride = q_head_stride; A.q_row_stride = q_row_stride; A.k_head_stride = k_head_stride; A.k_row_stride = k_row_stride;
  A.g = g; A.W = W; A.T = T; A.causal = causal ? 1 : 0; A.n_tiles = (T + OBS_KEYS - 1) / OBS_KEYS;
  A.BH = BH; A.extra_rows = (BH + A.n_tiles - 1) / A.n_tiles;
  const int64_t R = (int64_t)g * W;
  const int MB = (int)((R + OBS_ROWS - 1) / OBS_ROWS);
  A.part = scratch;
  A.ksq = A.part + (int64_t)BH * 2 * A.n_tiles * R * 2;
  A.stats = A.ksq + (int64_t)BH * A.n_tiles * 128;
  A.status = reinterpret_cast<int*>(A.stats + (int64_t)BH * R * 2);
  A.token = layer_token; A.channel = layer_channel;
  // the operands come by TMA when their layout can be mapped; a head's W query rows are one box,
  // which must start on a group of 8 rows and stay inside one 128-row block
  CUtensorMap tm_q, tm_k;
  memset(&tm_q, 0, sizeof(tm_q)); memset(&tm_k, 0, sizeof(tm_k));
  A.tma_k = obs_map(&tm_k, k, bf, k_head_stride, k_row_stride, BH, T, OBS_KEYS) ? 1 : 0;
  A.tma_q = (W % 8 == 0 && (R <= OBS_ROWS || OBS_ROWS % W == 0) &&
             obs_map(&tm_q, q_obs, bf, q_head_stride, q_row_stride, (int64_t)BH * g, W, W)) ? 1 : 0;
  const size_t smem = 1024 + (size_t)(1 + MB) * OBS_BLOCK;   // (the base is rounded up to 1024 bytes in the kernel)
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(A.status, 0, sizeof(int), st);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  const dim3 grid(A.n_tiles, BH);
  auto launch = [&](auto kern_stats, auto kern_reduce, auto kern_token) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern_stats, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern_token, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
    kern_stats<<<grid, OBS_THREADS, smem, st>>>(A, tm_q, tm_k);
    int rc = launch_status();
    if (rc != RDKV_OK) return rc;
    kern_reduce<<<dim3((unsigned)((R + OBS_RED_ROWS - 1) / OBS_RED_ROWS), BH), OBS_RED_THREADS, 0, st>>>(A);
    rc = launch_status();
    if (rc != RDKV_OK) return rc;
    kern_token<<<dim3(A.n_tiles, BH + A.extra_rows), OBS_THREADS, smem, st>>>(A, tm_q, tm_k);
    return launch_status();
  };
  if (bf) return launch(obs_tile_kernel<true, 0>, obs_reduce_kernel, obs_tile_kernel<true, 1>);
  return launch(obs_tile_kernel<false, 0>, obs_reduce_kernel, obs_tile_kernel<false, 1>);
}
