// Importance scores that feed the bit allocator, from the attention weights of the observation
// window (reference: obkv_fast.py:854-896 _score_one_layer, :208-246 apply_score_pooling).
//   token score   [B,H_kv,T]   = sum over the group's query heads and window positions of aw
//   channel score [B,H_kv,D]   = mean(q^2 over heads and window) * mean(k^2 over tokens)
//   pooling                      avg / max over a sliding window, zero or reflect padding
// All three are single passes over their inputs (HBM-bound).
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

// aw: [BH][R][T] (R = query heads of the group x window positions); out [BH][T]
__global__ void __launch_bounds__(256)
token_score_kernel(const void* __restrict__ aw, int dtype, int R, int T, float* __restrict__ out) {
  const int bh = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int64_t base = (int64_t)bh * R * T + t;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int r = 0;
  for (; r + 4 <= R; r += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] += load_any(aw, dtype, base + (int64_t)(r + u) * T);
  }
  for (; r < R; ++r) acc[0] += load_any(aw, dtype, base + (int64_t)r * T);
  out[(int64_t)bh * T + t] = round_to((acc[0] + acc[1]) + (acc[2] + acc[3]), dtype);
}

// partial sums of k^2 over a chunk of tokens: k [BH][T][D] -> part [BH][n_chunks][D]
constexpr int CH_THREADS = 256;
__global__ void __launch_bounds__(CH_THREADS)
channel_ksq_kernel(const void* __restrict__ k, int dtype, int T, int D, int64_t head_stride, int64_t row_stride,
                   int n_chunks, float* __restrict__ part) {
  extern __shared__ float s_part[];                        // [rows_par][D]
  const int bh = blockIdx.y, chunk = blockIdx.x;
  const int rows_par = CH_THREADS / D > 0 ? CH_THREADS / D : 1;
  const int c = threadIdx.x % D, rl = threadIdx.x / D;
  const int per = (T + n_chunks - 1) / n_chunks;
  const int t0 = chunk * per, t1 = min(T, t0 + per);
  float acc = 0.f;
  if (rl < rows_par && threadIdx.x < rows_par * D)
    for (int t = t0 + rl; t < t1; t += rows_par) {
      const float x = load_any(k, dtype, bh * head_stride + (int64_t)t * row_stride + c);
      acc = fmaf(x, x, acc);
    }
  if (threadIdx.x < rows_par * D) s_part[rl * D + c] = acc;
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
    for (int i = 0; i < rows_par; ++i) s += s_part[i * D + threadIdx.x];
    part[((int64_t)bh * n_chunks + chunk) * D + threadIdx.x] = s;
  }
}

// channel[bh][c] = mean_r(q[bh][r][c]^2) * (sum_chunks part)/T
__global__ void __launch_bounds__(128)
channel_final_kernel(const void* __restrict__ q, int q_dtype, int R, int D, const float* __restrict__ part,
                     int n_chunks, int T, float* __restrict__ out) {
  const int bh = blockIdx.x;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float qs = 0.f;
    for (int r = 0; r < R; ++r) {
      const float x = load_any(q, q_dtype, ((int64_t)bh * R + r) * D + c);
      qs = fmaf(x, x, qs);
    }
    float ks = 0.f;
    for (int i = 0; i < n_chunks; ++i) ks += part[((int64_t)bh * n_chunks + i) * D + c];
    out[(int64_t)bh * D + c] = (qs / (float)R) * (ks / (float)T);
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
  token_score_kernel<<<dim3((T + 255) / 256, BH), 256, 0, st>>>(aw, aw_dtype, R, T, layer_token);
  int rc = launch_status();
  if (rc != RDKV_OK) return rc;
  const int n_chunks = rdkv_score_chunks(T);
  const int rows_par = CH_THREADS / D > 0 ? CH_THREADS / D : 1;
  channel_ksq_kernel<<<dim3(n_chunks, BH), CH_THREADS, (size_t)rows_par * D * sizeof(float), st>>>(
      k, k_dtype, T, D, k_head_stride, k_row_stride, n_chunks, scratch);
  rc = launch_status();
  if (rc != RDKV_OK) return rc;
  channel_final_kernel<<<BH, 128, 0, st>>>(q, q_dtype, R, D, scratch, n_chunks, T, layer_channel);
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
