// Scores of one decode block for its recompression: how much attention the block's tokens get
// from a block of queries, and the per-channel statistic that ranks K channels.
//
// Replaces _score_block and _channel_score of the reference's blockwise decoder
// (obkv_accel/blockwise_decode.py:756-810):
//   token[h][t]   = sum over the head's g query heads and the Q query positions of
//                   softmax_t(q . k_t / sqrt(D))   (causal: position i sees keys t <= i)
//   channel[h][d] = mean_{g,Q}(q_d^2) * mean_t(k_d^2)
// One thread-block cluster of BS_CLUSTER CTAs per KV head (a decode block has 8 KV heads, far fewer
// than the GPU has SMs): every CTA holds the head's keys in shared memory as fp32 (rows padded by
// one word, so that lanes reading consecutive keys hit different banks) and takes every
// BS_CLUSTER-th group of (query head, position) pairs; a warp scores the keys one per lane,
// normalises across the warp and keeps its share of the column sums in registers.  The warps'
// shares are added in warp order inside a CTA, and the CTAs' sums in rank order by the cluster's
// first CTA, which reads them from the others' shared memory: the result repeats bit for bit.
#include <cooperative_groups.h>

#include "rdkv_common.cuh"

namespace rdkv {

constexpr int BS_THREADS = 256;
constexpr int BS_WARPS = BS_THREADS / 32;
constexpr int BS_MAX_T = 256;                    // keys of a block (the reference uses 64 or 128)
constexpr int BS_T_PER_LANE = BS_MAX_T / 32;
constexpr int BS_CLUSTER = 8;                    // CTAs per KV head (the portable cluster limit)

__global__ void __launch_bounds__(BS_THREADS)
block_score_kernel(const void* __restrict__ queries, int q_dtype, int64_t q_head_stride, int64_t q_pos_stride,
                   const void* __restrict__ keys, int k_dtype, int64_t k_head_stride, int64_t k_row_stride,
                   int g, int Q, int T, int Dh, int causal, float* __restrict__ token_out,
                   float* __restrict__ channel_out) {
  extern __shared__ float smem[];
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank(), csize = (int)cluster.num_blocks();
  const int h = blockIdx.x / csize, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ld = Dh + 1;
  const int span = T > Dh ? T : Dh;
  float* ks = smem;                                // [T][Dh + 1]
  float* qs = ks + (size_t)T * ld;                 // [BS_WARPS][Dh]: the pair a warp works on
  float* part = qs + BS_WARPS * Dh;                // [BS_WARPS][span]: the warps' shares
  float* mine = part + BS_WARPS * span;            // [2][span]: this CTA's token sums, q^2 sums
  for (int i = tid; i < T * Dh; i += BS_THREADS) {
    const int t = i / Dh, d = i % Dh;
    ks[t * ld + d] = load_q(keys, k_dtype, (int64_t)h * k_head_stride + (int64_t)t * k_row_stride + d);
  }
  __syncthreads();
  const float inv = 1.0f / sqrtf((float)Dh);
  float tok[BS_T_PER_LANE];
#pragma unroll
  for (int i = 0; i < BS_T_PER_LANE; ++i) tok[i] = 0.f;
  float qsq[4] = {0.f, 0.f, 0.f, 0.f};             // sums of q_d^2 for d = lane, lane + 32, ...
  float* myq = qs + warp * Dh;
  for (int pair = crank * BS_WARPS + warp; pair < g * Q; pair += csize * BS_WARPS) {
    const int gi = pair / Q, qi = pair % Q;
    const int64_t qoff = (int64_t)(h * g + gi) * q_head_stride + (int64_t)qi * q_pos_stride;
    __syncwarp();
    for (int d = lane, k = 0; d < Dh; d += 32, ++k) {
      const float x = load_q(queries, q_dtype, qoff + d);
      myq[d] = x;
      qsq[k] = fmaf(x, x, qsq[k]);
    }
    __syncwarp();
    if (token_out == nullptr) continue;            // channel statistic only
    float s[BS_T_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < BS_T_PER_LANE; ++i) {
      const int t = lane + 32 * i;
      float a = -INFINITY;
      if (t < T && !(causal && t > qi)) {
        a = 0.f;
        const float* kr = ks + t * ld;
        for (int d = 0; d < Dh; ++d) a = fmaf(myq[d], kr[d], a);
        a *= inv;
      }
      s[i] = a;
      mx = fmaxf(mx, a);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < BS_T_PER_LANE; ++i) {
      s[i] = s[i] == -INFINITY ? 0.f : expf(s[i] - mx);
      sum += s[i];
    }
    sum = warp_sum(sum);
    const float r = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < BS_T_PER_LANE; ++i) tok[i] = fmaf(s[i], r, tok[i]);
  }
  // this CTA's sums: the warps' shares, added in warp order
  if (token_out != nullptr) {
#pragma unroll
    for (int i = 0; i < BS_T_PER_LANE; ++i)
      if (lane + 32 * i < T) part[warp * span + lane + 32 * i] = tok[i];
    __syncthreads();
    for (int t = tid; t < T; t += BS_THREADS) {
      float a = 0.f;
      for (int w = 0; w < BS_WARPS; ++w) a += part[w * span + t];
      mine[t] = a;
    }
    __syncthreads();
  }
  for (int d = lane, k = 0; d < Dh; d += 32, ++k) part[warp * span + d] = qsq[k];
  __syncthreads();
  for (int d = tid; d < Dh; d += BS_THREADS) {
    float qa = 0.f;
    for (int w = 0; w < BS_WARPS; ++w) qa += part[w * span + d];
    mine[span + d] = qa;
  }
  cluster.sync();
  // the cluster's first CTA adds the CTAs' sums in rank order
  if (crank == 0) {
    if (token_out != nullptr)
      for (int t = tid; t < T; t += BS_THREADS) {
        float a = 0.f;
        for (int r = 0; r < csize; ++r) a += cluster.map_shared_rank(mine, r)[t];
        token_out[(int64_t)h * T + t] = a;
      }
    for (int d = tid; d < Dh; d += BS_THREADS) {
      float qa = 0.f;
      for (int r = 0; r < csize; ++r) qa += cluster.map_shared_rank(mine, r)[span + d];
      float ka = 0.f;
      for (int t = 0; t < T; ++t) ka = fmaf(ks[t * ld + d], ks[t * ld + d], ka);
      channel_out[(int64_t)h * Dh + d] = (qa / (float)(g * Q)) * (ka / (float)T);
    }
  }
  cluster.sync();                                  // the others' shared memory stays until it was read
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int rdkv_block_scores(const void* queries, int q_dtype, int64_t q_head_stride, int64_t q_pos_stride,
                                 const void* keys, int k_dtype, int64_t k_head_stride, int64_t k_row_stride,
                                 int H_kv, int g, int Q, int T, int D, int causal, float* token_out,
                                 float* channel_out, void* stream) {
  if (queries == nullptr || keys == nullptr || channel_out == nullptr) return RDKV_ERR_BAD_ARG;
  if (q_dtype < RDKV_F16 || q_dtype > RDKV_F32 || k_dtype < RDKV_F16 || k_dtype > RDKV_F32) return RDKV_ERR_BAD_ARG;
  if (H_kv < 0 || g <= 0 || Q <= 0 || T <= 0 || D <= 0) return RDKV_ERR_BAD_ARG;
  if (D > 128 || T > BS_MAX_T) return RDKV_ERR_TOO_LARGE;
  if (causal && Q != T) return RDKV_ERR_BAD_SHAPE;
  if (H_kv == 0) return RDKV_OK;
  const int span = T > D ? T : D;
  const size_t smem =
      sizeof(float) * ((size_t)T * (D + 1) + (size_t)BS_WARPS * D + (size_t)BS_WARPS * span + 2 * (size_t)span);
  cudaError_t e = cudaFuncSetAttribute(block_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(H_kv * BS_CLUSTER);
  cfg.blockDim = dim3(BS_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = BS_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, block_score_kernel, queries, q_dtype, q_head_stride, q_pos_stride, keys, k_dtype,
                         k_head_stride, k_row_stride, g, Q, T, D, causal, token_out, channel_out);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  return launch_status();
}
