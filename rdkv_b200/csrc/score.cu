// Importance scores that feed the bit allocator, from the attention weights of the observation
// window (reference: obkv_fast.py:854-896 _score_one_layer, :208-246 apply_score_pooling).
//   token score   [B,H_kv,T]   = sum over the group's query heads and window positions of aw
//   channel score [B,H_kv,D]   = mean(q^2 over heads and window) * mean(k^2 over tokens)
//   pooling                      avg / max over a sliding window, zero or reflect padding
// Token and channel scores come from one launch; all passes read their inputs once (HBM-bound).
#include "rdkv_common.cuh"

namespace rdkv {

__device__ __forceinline__ float load_any(const void* p, int dtype, int64_t i) {
  if (dtype == RDKV_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  if (dtype == RDKV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

// Rounds an fp32 sum to the precision the reference's `aw.sum(...)` result has (aw's own dtype).
__device__ __forceinline__ float round_to(float x, int dtype) {
  if (dtype == RDKV_F16) return __half2float(__float2half_rn(x));
  if (dtype == RDKV_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}

// One launch scores a layer.  Block columns [0, n_tok) sum the attention weights of 512 tokens
// over the R rows of the window; block columns [n_tok, n_tok + n_chunks) sum k^2 over a chunk of
// tokens into part [BH][n_chunks][D], and the chunk block that arrives last for its head (a counter
// per head, zeroed by the entry point) adds the chunks in chunk order, sums q^2 over the window
// and writes the channel score.  Every sum runs in a fixed order, so results repeat bit for bit.
//   aw [BH][R][T] -> token [BH][T];  k [BH][T][D], q [BH][R][D] -> channel [BH][D]
constexpr int SC_THREADS = 256;
constexpr int SC_VEC_SMEM = 16384;                      // shared memory of the vectorised k^2 pass: [row lanes][D] fp32
__global__ void __launch_bounds__(SC_THREADS)
score_layer_kernel(const void* __restrict__ aw, int aw_dtype, const void* __restrict__ q, int q_dtype,
                   const void* __restrict__ k, int k_dtype, int64_t head_stride, int64_t row_stride, int R, int T,
                   int D, int n_tok, int n_chunks, float* __restrict__ part, unsigned* __restrict__ arrived,
                   float* __restrict__ token_out, float* __restrict__ channel_out) {
  extern __shared__ float s_part[];                        // [rows_par][D], used twice by the last block
  __shared__ int s_last;
  const int bh = blockIdx.y, tid = threadIdx.x;
  if ((int)blockIdx.x < n_tok) {
    // 512 tokens per block: a thread sums two adjacent tokens (one 32-bit load per row for 16-bit
    // weights), eight rows in flight; per token the rows are added in a fixed order
    const int t = (blockIdx.x * SC_THREADS + tid) * 2;
    if (t >= T) return;
    const int64_t base = (int64_t)bh * R * T + t;
    const bool pair = aw_dtype != RDKV_F32 && (T & 1) == 0 && (reinterpret_cast<uintptr_t>(aw) & 3) == 0;
    float a0[8], a1[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) a0[u] = a1[u] = 0.f;
    int r = 0;
    if (pair) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(aw) + base);
      const int64_t row_words = T >> 1;
      for (; r + 8 <= R; r += 8) {
        uint32_t x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) x[u] = __ldg(w + (int64_t)(r + u) * row_words);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (aw_dtype == RDKV_F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&x[u]));
            a0[u] += f.x; a1[u] += f.y;
          } else {
            a0[u] += __uint_as_float(x[u] << 16); a1[u] += __uint_as_float(x[u] & 0xFFFF0000u);
          }
        }
      }
    }
    const bool two = t + 1 < T;
    for (; r < R; ++r) {
      a0[r & 7] += load_any(aw, aw_dtype, base + (int64_t)r * T);
      if (two) a1[r & 7] += load_any(aw, aw_dtype, base + (int64_t)r * T + 1);
    }
    token_out[(int64_t)bh * T + t] =
        round_to(((a0[0] + a0[1]) + (a0[2] + a0[3])) + ((a0[4] + a0[5]) + (a0[6] + a0[7])), aw_dtype);
    if (two)
      token_out[(int64_t)bh * T + t + 1] =
          round_to(((a1[0] + a1[1]) + (a1[2] + a1[3])) + ((a1[4] + a1[5]) + (a1[6] + a1[7])), aw_dtype);
    return;
  }
  const int chunk = blockIdx.x - n_tok;
  const int rows_par = SC_THREADS / D > 0 ? SC_THREADS / D : 1;
  const bool on = tid < rows_par * D;
  const int c = tid % D, rl = tid / D;
  const int per = (T + n_chunks - 1) / n_chunks;
  const int t0 = chunk * per, t1 = min(T, t0 + per);
  float acc = 0.f;
  const int lanes_row = D >> 3;                            // threads per row at eight channels each
  const bool vec = k_dtype != RDKV_F32 && (D & 7) == 0 && SC_THREADS % lanes_row == 0 && (row_stride & 7) == 0 &&
                   (head_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(k) & 15) == 0 &&
                   SC_THREADS / lanes_row * D * (int)sizeof(float) <= SC_VEC_SMEM;
  if (vec) {
    // 16-byte loads: thread (row lane, channel octet) sums the squares of its eight channels over
    // every rows_v-th token, four rows in flight; the row lanes are then added in lane order
    const int rows_v = SC_THREADS / lanes_row, o8 = (tid % lanes_row) * 8, rv = tid / lanes_row;
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const uint16_t* kb = reinterpret_cast<const uint16_t*>(k) + bh * head_stride + o8;
    auto add = [&](const uint4& x) {
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float lo, hi;
        if (k_dtype == RDKV_F16) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
          lo = f.x; hi = f.y;
        } else {
          lo = __uint_as_float(w[i] << 16); hi = __uint_as_float(w[i] & 0xFFFF0000u);
        }
        a[2 * i] = fmaf(lo, lo, a[2 * i]); a[2 * i + 1] = fmaf(hi, hi, a[2 * i + 1]);
      }
    };
    int t = t0 + rv;
    for (; t + 3 * rows_v < t1; t += 4 * rows_v) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) x[u] = __ldg(reinterpret_cast<const uint4*>(kb + (int64_t)(t + u * rows_v) * row_stride));
#pragma unroll
      for (int u = 0; u < 4; ++u) add(x[u]);
    }
    for (; t < t1; t += rows_v) add(__ldg(reinterpret_cast<const uint4*>(kb + (int64_t)t * row_stride)));
    float* sv = s_part;                                    // [rows_v][D]
#pragma unroll
    for (int i = 0; i < 8; ++i) sv[rv * D + o8 + i] = a[i];
    __syncthreads();
    if (tid < D) {
      float s = 0.f;
      for (int i = 0; i < rows_v; ++i) s += sv[i * D + tid];
      part[((int64_t)bh * n_chunks + chunk) * D + tid] = s;
      __threadfence();
    }
    __syncthreads();
  } else {
  if (on)
    for (int t = t0 + rl; t < t1; t += rows_par) {
      const float x = load_any(k, k_dtype, bh * head_stride + (int64_t)t * row_stride + c);
      acc = fmaf(x, x, acc);
    }
  if (on) s_part[rl * D + c] = acc;
  __syncthreads();
  if (tid < D) {
    float s = 0.f;
    for (int i = 0; i < rows_par; ++i) s += s_part[i * D + tid];
    part[((int64_t)bh * n_chunks + chunk) * D + tid] = s;
    __threadfence();
  }
  __syncthreads();
  }
  if (tid == 0) s_last = atomicAdd(&arrived[bh], 1u) == (unsigned)(n_chunks - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the head's last chunk block: slices of the window rows and of the chunks per thread row
  float qs = 0.f, ks = 0.f;
  if (on) {
    for (int r = rl; r < R; r += rows_par) {
      const float x = load_any(q, q_dtype, ((int64_t)bh * R + r) * D + c);
      qs = fmaf(x, x, qs);
    }
    for (int i = rl; i < n_chunks; i += rows_par) ks += __ldcg(part + ((int64_t)bh * n_chunks + i) * D + c);
  }
  float qsum = 0.f, ksum = 0.f;
  if (on) s_part[rl * D + c] = qs;
  __syncthreads();
  if (tid < D)
    for (int i = 0; i < rows_par; ++i) qsum += s_part[i * D + tid];
  __syncthreads();
  if (on) s_part[rl * D + c] = ks;
  __syncthreads();
  if (tid < D) {
    for (int i = 0; i < rows_par; ++i) ksum += s_part[i * D + tid];
    channel_out[(int64_t)bh * D + tid] = (qsum / (float)R) * (ksum / (float)T);
  }
}

// Sliding-window pooling of rows of fp32 scores, stride 1.  Zero padding: kernel_size taps, taps
// outside the row count as 0 (avg, divisor kernel_size) or are skipped (max).  Reflect padding:
// min(kernel_size, 2*len-1) taps around i, indices mirrored at the ends.  The taps are added in
// ascending order and divided once, as torch's avg_pool1d does.
__global__ void __launch_bounds__(256)
pool_kernel(const float* __restrict__ in, int64_t in_stride, int len, int out_len, int ksize, int pad, int is_max,
            int reflect, float* __restrict__ out, int64_t out_stride) {
  const int row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= out_len) return;
  const float* x = in + row * in_stride;
  float acc = is_max ? -INFINITY : 0.f;
  for (int w = 0; w < ksize; ++w) {
    int j = i - pad + w;
    if (reflect) {
      if (j < 0) j = -j;
      if (j >= len) j = 2 * (len - 1) - j;
    }
    if (j < 0 || j >= len) continue;                        // zero padding: contributes 0 / is not a candidate
    acc = is_max ? fmaxf(acc, x[j]) : acc + x[j];
  }
  out[row * out_stride + i] = is_max ? acc : acc / (float)ksize;
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int rdkv_score_chunks(int T) {
  int n = (T + 511) / 512;
  return n < 1 ? 1 : (n > 256 ? 256 : n);
}

extern "C" int64_t rdkv_score_scratch_words(int BH, int T, int D) {
  if (BH < 0 || T <= 0 || D <= 0) return 0;
  return (int64_t)BH * rdkv_score_chunks(T) * D + BH;
}

extern "C" int rdkv_score_layer(const void* aw, int aw_dtype, const void* q, int q_dtype, const void* k, int k_dtype,
                                int64_t k_head_stride, int64_t k_row_stride, int BH, int R, int T, int D,
                                float* scratch, float* layer_token, float* layer_channel, void* stream) {
  if (aw == nullptr || q == nullptr || k == nullptr || layer_token == nullptr || layer_channel == nullptr ||
      scratch == nullptr)
    return RDKV_ERR_BAD_ARG;
  if (BH < 0 || R <= 0 || T <= 0 || D <= 0 || D > 256) return RDKV_ERR_BAD_SHAPE;
  for (int dt : {aw_dtype, q_dtype, k_dtype})
    if (dt < RDKV_F16 || dt > RDKV_F32) return RDKV_ERR_BAD_ARG;
  if (BH == 0) return RDKV_OK;
  if (BH > 65535) return RDKV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const int n_chunks = rdkv_score_chunks(T);
  const int n_tok = (T + 2 * SC_THREADS - 1) / (2 * SC_THREADS);
  const int rows_par = SC_THREADS / D > 0 ? SC_THREADS / D : 1;
  size_t smem = (size_t)rows_par * D * sizeof(float);
  if (smem < (size_t)SC_VEC_SMEM) smem = SC_VEC_SMEM;
  unsigned* arrived = reinterpret_cast<unsigned*>(scratch + (int64_t)BH * n_chunks * D);
  cudaError_t e = cudaMemsetAsync(arrived, 0, sizeof(unsigned) * BH, st);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  score_layer_kernel<<<dim3(n_tok + n_chunks, BH), SC_THREADS, smem, st>>>(
      aw, aw_dtype, q, q_dtype, k, k_dtype, k_head_stride, k_row_stride, R, T, D, n_tok, n_chunks, scratch, arrived,
      layer_token, layer_channel);
  return launch_status();
}

extern "C" int rdkv_score_pool(const float* scores, int64_t row_stride, int rows, int len, int pool_max,
                               int kernel_size, int reflect, float* out, int64_t out_row_stride, int out_len,
                               void* stream) {
  if (scores == nullptr || out == nullptr || rows < 0 || len <= 0 || kernel_size <= 0) return RDKV_ERR_BAD_ARG;
  int ksize = kernel_size;
  if (reflect) ksize = kernel_size < 2 * len - 1 ? kernel_size : 2 * len - 1;
  const int pad = ksize / 2;
  if (out_len != len + 2 * pad - ksize + 1) return RDKV_ERR_BAD_SHAPE;
  if (rows == 0) return RDKV_OK;
  if (rows > 65535) return RDKV_ERR_TOO_LARGE;
  pool_kernel<<<dim3((out_len + 255) / 256, rows), 256, 0, (cudaStream_t)stream>>>(
      scores, row_stride, len, out_len, ksize, pad, pool_max ? 1 : 0, reflect ? 1 : 0, out, out_row_stride);
  return launch_status();
}
