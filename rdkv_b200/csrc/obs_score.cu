// Importance scores of a prefilled layer straight from the observation window's queries and the
// layer's keys, without the [H_q, W, T] attention weights ever reaching memory.
//
// Replaces the scoring step of the reference's prefill (obkv_fast.py:1443-1466): attention weights
// of the last W query positions over all T keys (matmul in the model's 16-bit type, scaled, causal
// mask, softmax), then _score_one_layer (:854-896): token score [H_kv][T] = sum of the weights
// over the head's g query heads and the W positions, channel score [H_kv][128] = mean(q^2) *
// mean_t(k^2).  The reference materialises the weights (2 bytes x H_q x W x T) and reads them
// back; here every tile of scores lives in registers.
//
// Three launches per layer:
//   obs_stats_kernel   per (KV head, 128-key tile): S = Q.K^T on the tensor cores (rows = (query
//                      head, position) pairs, 16 per MMA), rounded as the reference's 16-bit
//                      matmul and scaling round it, masked; per row the tile's maximum and
//                      sum of exponentials; per channel the tile's sum of k^2.
//   obs_reduce_kernel  per KV head: the rows' maxima and sums over all tiles; the channel score.
//   obs_token_kernel   per (KV head, tile): the same scores again, p = exp(s - M) / L rounded to
//                      the 16-bit type, summed over the rows: the token scores of the tile.
// The keys are read twice (the second time mostly from L2); sums run in a fixed order.
#include "rdkv_common.cuh"

namespace rdkv {

constexpr int OBS_THREADS = 256;
constexpr int OBS_WARPS = OBS_THREADS / 32;
constexpr int OBS_KEYS = 128;                    // keys per tile
constexpr int OBS_LD = 136;                      // padded row length in shared memory (16-bit elements): ldmatrix rows hit distinct banks
constexpr int OBS_MAX_ROWS = 256;                // (query head, position) pairs per KV head

__device__ __forceinline__ uint32_t obs_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <bool BF16>
__device__ __forceinline__ void obs_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

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

// 16-byte chunks of `rows` rows of 128 16-bit elements (row stride given in elements) into padded
// shared memory; rows >= rows_valid are zero-filled.
__device__ __forceinline__ void obs_stage(uint16_t* dst, const uint16_t* src, int64_t row_stride, int rows, int rows_valid,
                                          bool aligned) {
  for (int i = threadIdx.x; i < rows * 16; i += OBS_THREADS) {
    const int row = i >> 4, c = (i & 15) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_valid) {
      const uint16_t* p = src + (int64_t)row * row_stride + c;
      if (aligned) v = *reinterpret_cast<const uint4*>(p);
      else {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) w[e] = (uint32_t)p[2 * e] | (uint32_t)p[2 * e + 1] << 16;
        v = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    *reinterpret_cast<uint4*>(dst + row * OBS_LD + c) = v;
  }
}

// The shared part of both passes: the scores of m-tile `mt` (16 rows) against key group `nt` (8 keys)
// of the staged tile, rounded as the reference rounds them (the 16-bit matmul result, then its
// product with 1/sqrt(128) in the same type).  a[ks]: the m-tile's query fragments.
template <bool BF16>
__device__ __forceinline__ void obs_scores(float (&s)[4], const uint32_t (&a)[8][4], uint32_t k_tile, int nt, int lane) {
  float c[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};   // two chains of four MMAs
  const uint32_t base = k_tile + (uint32_t)((nt * 8 + (lane & 7)) * OBS_LD + 8 * (lane >> 3)) * 2u;
#pragma unroll
  for (int kp = 0; kp < 4; ++kp) {                           // two 16-channel steps per ldmatrix.x4
    uint32_t b[4];
    ldm_x4(b, base + (uint32_t)kp * 64u);
    obs_mma<BF16>(c, a[2 * kp], b[0], b[1]);
    obs_mma<BF16>(d, a[2 * kp + 1], b[2], b[3]);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) s[e] = obs_round<BF16>(obs_round<BF16>(c[e] + d[e]) * INV_SQRT_D);
}

struct ObsArgs {
  const uint16_t* q; const uint16_t* k;
  int64_t q_head_stride, q_row_stride, k_head_stride, k_row_stride;   // elements
  int g, W, T, causal, n_tiles;
  float* part;         // [BH][n_tiles][R][2] tile maxima and sums
  float* ksq;          // [BH][n_tiles][128] tile sums of k^2
  float* stats;        // [BH][R][2] maxima and sums over all keys
  float* token;        // [BH][T]
  float* channel;      // [BH][128]
};

// PASS 0: row statistics and k^2 sums of a tile.  PASS 1: token scores of a tile.
template <bool BF16, int PASS>
__global__ void __launch_bounds__(OBS_THREADS, 3)
obs_tile_kernel(ObsArgs A) {
  extern __shared__ __align__(16) unsigned char obs_raw[];
  const int tile = blockIdx.x, bh = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = lane >> 2, j = lane & 3;
  const int R = A.g * A.W, T = A.T;
  const int rows_pad = (R + 15) & ~15;
  uint16_t* s_q = reinterpret_cast<uint16_t*>(obs_raw);               // [rows_pad][OBS_LD]
  uint16_t* s_k = s_q + (size_t)rows_pad * OBS_LD;                     // [OBS_KEYS][OBS_LD]
  float* s_col = reinterpret_cast<float*>(s_k + (size_t)OBS_KEYS * OBS_LD);   // [OBS_WARPS][OBS_KEYS] (PASS 1)
  const int t0 = tile * OBS_KEYS, n_keys = min(OBS_KEYS, T - t0);
  const uint16_t* kt = A.k + bh * A.k_head_stride + (int64_t)t0 * A.k_row_stride;
  const bool k_al = (A.k_row_stride & 7) == 0 && (A.k_head_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(A.k) & 15) == 0;
  const bool q_al = (A.q_row_stride & 7) == 0 && (A.q_head_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(A.q) & 15) == 0;
  obs_stage(s_k, kt, A.k_row_stride, OBS_KEYS, n_keys, k_al);
  for (int gi = 0; gi < A.g; ++gi)                           // row gi*W + w = query head gi of the group, window position w
    obs_stage(s_q + (size_t)gi * A.W * OBS_LD, A.q + ((int64_t)bh * A.g + gi) * A.q_head_stride, A.q_row_stride, A.W, A.W, q_al);
  for (int i = tid; i < (rows_pad - R) * 16; i += OBS_THREADS)   // pad rows of the last m-tile
    *reinterpret_cast<uint4*>(s_q + (size_t)(R + (i >> 4)) * OBS_LD + (i & 15) * 8) = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();

  if (PASS == 0) {                                           // k^2 of the tile: thread = (half of the keys, channel)
    const int c = tid & 127, half = tid >> 7;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int t = half * (OBS_KEYS / 2); t < (half + 1) * (OBS_KEYS / 2); ++t) {   // (rows past the tile's keys are zeros)
      const uint16_t b = s_k[t * OBS_LD + c];
      const float x = BF16 ? __uint_as_float((uint32_t)b << 16) : h2f(b);
      acc[t & 3] = fmaf(x, x, acc[t & 3]);
    }
    s_col[half * 128 + c] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    __syncthreads();
    if (tid < 128) A.ksq[((int64_t)bh * A.n_tiles + tile) * 128 + tid] = s_col[tid] + s_col[128 + tid];
  }

  const uint32_t q32 = obs_smem(s_q), k32 = obs_smem(s_k);
  if (PASS == 1) {                                           // the warps' column sums start at zero
    for (int i = tid; i < OBS_WARPS * OBS_KEYS; i += OBS_THREADS) s_col[i] = 0.f;
    __syncthreads();
  }
  for (int mt = warp; mt * 16 < R; mt += OBS_WARPS) {
    uint32_t a[8][4];
    {
      const uint32_t base = q32 + (uint32_t)((mt * 16 + (lane & 15)) * OBS_LD + 8 * (lane >> 4)) * 2u;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) ldm_x4(a[ks], base + (uint32_t)ks * 32u);
    }
    // rows r and r + 8 of the m-tile: their window positions decide which keys they may see
    const int row_a = mt * 16 + r, row_b = row_a + 8;
    const int lim_a = A.causal ? T - A.W + (row_a % A.W) : T - 1;       // last visible key
    const int lim_b = A.causal ? T - A.W + (row_b % A.W) : T - 1;
    // (only tiles that reach into the window or past the sequence's end have anything to mask)
    const bool edge = t0 + OBS_KEYS > (A.causal ? T - A.W : T);
    if (PASS == 0) {
      // half a tile at a time: its scores, the rows' maxima over the half, one exponential each; the
      // two halves merge like two tiles
      float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        constexpr int NH = OBS_KEYS / 16;
        float sc[NH][4];
#pragma unroll
        for (int i = 0; i < NH; ++i) {
          const int nt = hf * NH + i;
          obs_scores<BF16>(sc[i], a, k32, nt, lane);
          if (edge) {
            const int t = t0 + nt * 8 + 2 * j;
            if (t > lim_a) sc[i][0] = -INFINITY;
            if (t + 1 > lim_a) sc[i][1] = -INFINITY;
            if (t > lim_b) sc[i][2] = -INFINITY;
            if (t + 1 > lim_b) sc[i][3] = -INFINITY;
          }
        }
        float h_a = -INFINITY, h_b = -INFINITY;
#pragma unroll
        for (int i = 0; i < NH; ++i) {
          h_a = fmaxf(h_a, fmaxf(sc[i][0], sc[i][1])); h_b = fmaxf(h_b, fmaxf(sc[i][2], sc[i][3]));
        }
        const float n_a = fmaxf(m_a, h_a), n_b = fmaxf(m_b, h_b);
        const float ca = n_a > -INFINITY ? n_a * OBS_LOG2E : 0.f, cb = n_b > -INFINITY ? n_b * OBS_LOG2E : 0.f;
        float s_a = 0.f, s_b = 0.f;
#pragma unroll
        for (int i = 0; i < NH; ++i) {                       // (2^-inf = 0: masked keys add nothing)
          s_a += obs_ex2(fmaf(sc[i][0], OBS_LOG2E, -ca)) + obs_ex2(fmaf(sc[i][1], OBS_LOG2E, -ca));
          s_b += obs_ex2(fmaf(sc[i][2], OBS_LOG2E, -cb)) + obs_ex2(fmaf(sc[i][3], OBS_LOG2E, -cb));
        }
        l_a = (m_a > -INFINITY ? l_a * obs_ex2(fmaf(m_a, OBS_LOG2E, -ca)) : 0.f) + s_a;
        l_b = (m_b > -INFINITY ? l_b * obs_ex2(fmaf(m_b, OBS_LOG2E, -cb)) : 0.f) + s_b;
        m_a = n_a; m_b = n_b;
      }
      // the four threads of a quad hold the same rows: merge their (m, l) along a fixed tree
#pragma unroll
      for (int o = 1; o < 4; o <<= 1) {
        const float om_a = __shfl_xor_sync(0xffffffffu, m_a, o), ol_a = __shfl_xor_sync(0xffffffffu, l_a, o);
        const float om_b = __shfl_xor_sync(0xffffffffu, m_b, o), ol_b = __shfl_xor_sync(0xffffffffu, l_b, o);
        const float na = fmaxf(m_a, om_a), nb = fmaxf(m_b, om_b);
        l_a = na > -INFINITY ? l_a * obs_ex2((m_a - na) * OBS_LOG2E) + ol_a * obs_ex2((om_a - na) * OBS_LOG2E) : 0.f;
        l_b = nb > -INFINITY ? l_b * obs_ex2((m_b - nb) * OBS_LOG2E) + ol_b * obs_ex2((om_b - nb) * OBS_LOG2E) : 0.f;
        m_a = na; m_b = nb;
      }
      if (j == 0) {
        float* dst = A.part + (((int64_t)bh * A.n_tiles + tile) * R) * 2;
        if (row_a < R) { dst[2 * row_a] = m_a; dst[2 * row_a + 1] = l_a; }
        if (row_b < R) { dst[2 * row_b] = m_b; dst[2 * row_b + 1] = l_b; }
      }
    } else {
      const float* st = A.stats + (int64_t)bh * R * 2;
      const float M_a = row_a < R ? st[2 * row_a] : 0.f, L_a = row_a < R ? st[2 * row_a + 1] : 1.f;
      const float M_b = row_b < R ? st[2 * row_b] : 0.f, L_b = row_b < R ? st[2 * row_b + 1] : 1.f;
      const float ca = M_a * OBS_LOG2E, cb = M_b * OBS_LOG2E;
      const float ia = row_a < R ? __frcp_rn(L_a) : 0.f, ib = row_b < R ? __frcp_rn(L_b) : 0.f;   // (a row past R weighs nothing)
#pragma unroll 4
      for (int nt = 0; nt < OBS_KEYS / 8; ++nt) {
        float s[4];
        obs_scores<BF16>(s, a, k32, nt, lane);
        if (edge) {
          const int t = t0 + nt * 8 + 2 * j;
          if (t > lim_a) s[0] = -INFINITY;
          if (t + 1 > lim_a) s[1] = -INFINITY;
          if (t > lim_b) s[2] = -INFINITY;
          if (t + 1 > lim_b) s[3] = -INFINITY;
        }
        // p = exp(s - M) / L in fp32, rounded to the 16-bit type as the reference's softmax output is
        const float p0 = obs_round<BF16>(obs_ex2(fmaf(s[0], OBS_LOG2E, -ca)) * ia);
        const float p1 = obs_round<BF16>(obs_ex2(fmaf(s[1], OBS_LOG2E, -ca)) * ia);
        const float p2 = obs_round<BF16>(obs_ex2(fmaf(s[2], OBS_LOG2E, -cb)) * ib);
        const float p3 = obs_round<BF16>(obs_ex2(fmaf(s[3], OBS_LOG2E, -cb)) * ib);
        // column sums over the m-tile's rows (lanes with the same j), added to the warp's own line
        float c0 = p0 + p2, c1 = p1 + p3;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          c0 += __shfl_xor_sync(0xffffffffu, c0, o); c1 += __shfl_xor_sync(0xffffffffu, c1, o);
        }
        if (r == 0) {
          float* dst = s_col + warp * OBS_KEYS + nt * 8 + 2 * j;
          dst[0] += c0; dst[1] += c1;
        }
      }
    }
  }
  if (PASS == 1) {
    // the warps' lines are added in warp order
    __syncthreads();
    if (tid < n_keys) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < OBS_WARPS; ++w) v += s_col[w * OBS_KEYS + tid];
      A.token[(int64_t)bh * T + t0 + tid] = obs_round<BF16>(v);      // (the reference's aw.sum(...) is in aw's type)
    }
  }
}

// Per KV head: the rows' maxima and sums over all tiles, and the channel score.  blockIdx.y <
// OBS_RED_ROWS takes an eighth of the rows, a warp per row: the lanes take every 32nd tile, then
// merge their (m, l) pairs along a fixed tree; the last blockIdx.y takes the channels.
constexpr int OBS_RED_ROWS = 8;
template <bool BF16>
__global__ void __launch_bounds__(256)
obs_reduce_kernel(ObsArgs A) {
  const int bh = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int R = A.g * A.W;
  if ((int)blockIdx.y < OBS_RED_ROWS) {
    const int per = (R + OBS_RED_ROWS - 1) / OBS_RED_ROWS;
    const int r_end = min(R, ((int)blockIdx.y + 1) * per);
    for (int row = blockIdx.y * per + warp; row < r_end; row += 8) {
      const float* p = A.part + ((int64_t)bh * A.n_tiles * R + row) * 2;
      float M = -INFINITY, L = 0.f;
      for (int i = lane; i < A.n_tiles; i += 32) {
        const float2 ml = *reinterpret_cast<const float2*>(p + (int64_t)i * R * 2);
        if (ml.x > -INFINITY) {
          const float n = fmaxf(M, ml.x);
          L = L * obs_ex2((M - n) * OBS_LOG2E) + ml.y * obs_ex2((ml.x - n) * OBS_LOG2E);
          M = n;
        }
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, M, o), ol = __shfl_xor_sync(0xffffffffu, L, o);
        const float n = fmaxf(M, om);
        L = n > -INFINITY ? L * obs_ex2((M - n) * OBS_LOG2E) + ol * obs_ex2((om - n) * OBS_LOG2E) : 0.f;
        M = n;
      }
      if (lane == 0) {
        A.stats[((int64_t)bh * R + row) * 2] = M;
        A.stats[((int64_t)bh * R + row) * 2 + 1] = L;
      }
    }
    return;
  }
  // channel score: threads (half, channel) sum every other row / tile, the halves are added at the end
  __shared__ float s_q2[2][128], s_k2[2][128];
  const int c = tid & 127, half = tid >> 7;
  float qs = 0.f, ks = 0.f;
#pragma unroll 4
  for (int row = half; row < R; row += 2) {
    const uint16_t b = A.q[((int64_t)bh * A.g + row / A.W) * A.q_head_stride + (int64_t)(row % A.W) * A.q_row_stride + c];
    const float x = BF16 ? __uint_as_float((uint32_t)b << 16) : h2f(b);
    qs = fmaf(x, x, qs);
  }
#pragma unroll 8
  for (int i = half; i < A.n_tiles; i += 2) ks += A.ksq[((int64_t)bh * A.n_tiles + i) * 128 + c];
  s_q2[half][c] = qs; s_k2[half][c] = ks;
  __syncthreads();
  if (tid < 128)
    A.channel[(int64_t)bh * 128 + tid] = ((s_q2[0][tid] + s_q2[1][tid]) / (float)R) * ((s_k2[0][tid] + s_k2[1][tid]) / (float)A.T);
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int64_t rdkv_obs_scratch_words(int BH, int g, int W, int T) {
  if (BH < 0 || g <= 0 || W <= 0 || T <= 0) return 0;
  const int64_t n_tiles = (T + OBS_KEYS - 1) / OBS_KEYS, R = (int64_t)g * W;
  return BH * (n_tiles * R * 2 + n_tiles * 128 + R * 2);
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
  if (BH > 65535) return RDKV_ERR_TOO_LARGE;
  ObsArgs A;
  A.q = reinterpret_cast<const uint16_t*>(q_obs); A.k = reinterpret_cast<const uint16_t*>(k);
  A.q_head_stride = q_head_stride; A.q_row_stride = q_row_stride; A.k_head_stride = k_head_stride; A.k_row_stride = k_row_stride;
  A.g = g; A.W = W; A.T = T; A.causal = causal ? 1 : 0; A.n_tiles = (T + OBS_KEYS - 1) / OBS_KEYS;
  const int64_t R = (int64_t)g * W;
  A.part = scratch;
  A.ksq = A.part + (int64_t)BH * A.n_tiles * R * 2;
  A.stats = A.ksq + (int64_t)BH * A.n_tiles * 128;
  A.token = layer_token; A.channel = layer_channel;
  const int rows_pad = ((int)R + 15) & ~15;
  const size_t smem = (size_t)(rows_pad + OBS_KEYS) * OBS_LD * 2 + (size_t)OBS_WARPS * OBS_KEYS * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(A.n_tiles, BH);
  const bool bf = dtype == RDKV_BF16;
  auto launch = [&](auto kern_stats, auto kern_reduce, auto kern_token) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern_stats, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern_token, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
    kern_stats<<<grid, OBS_THREADS, smem, st>>>(A);
    int rc = launch_status();
    if (rc != RDKV_OK) return rc;
    kern_reduce<<<dim3(BH, OBS_RED_ROWS + 1), 256, 0, st>>>(A);
    rc = launch_status();
    if (rc != RDKV_OK) return rc;
    kern_token<<<grid, OBS_THREADS, smem, st>>>(A);
    return launch_status();
  };
  if (bf) return launch(obs_tile_kernel<true, 0>, obs_reduce_kernel<true>, obs_tile_kernel<true, 1>);
  return launch(obs_tile_kernel<false, 0>, obs_reduce_kernel<false>, obs_tile_kernel<false, 1>);
}
