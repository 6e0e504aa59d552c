// Packed-KV decode attention, two-stage operators: K-side scores, V-side weighted
// sum, and the log-sum-exp combine of split-sequence partial records.
//
// Math follows the reference's kernels (obkv_accel/triton_k_kernel.py:14-16 "bias
// trick"; obkv_accel/triton_v_kernel.py:1-31 layouts): scale is folded into q
// (K side) or into the softmax weight (V side) so the inner loops touch raw
// integer codes; the zero-point term is subtracted once per row.
#include "rdkv_common.cuh"

namespace rdkv {

thread_local int g_last_cuda_error = 0;

constexpr int SCORE_THREADS = 128;
constexpr int GP = 8;                 // query heads handled per register pass

// qs[hq][slot] = q[hq][perm[slot]] * scale[slot]; bias[hq] = sum_slot zp*qs.
// Called by all threads of the block; smem_qs holds g*d_pad floats, smem_bias g floats,
// smem_red at least (blockDim.x/32)*g floats.
__device__ void setup_q(const rdkv_layer_view& v, int h, int g, int d_pad, const void* q, int q_dtype,
                        int64_t q_head0_off, int64_t q_row_stride, float* smem_qs, float* smem_bias,
                        float* smem_red) {
  const uint16_t* sc = v.k_scale + (int64_t)h * d_pad;
  const uint16_t* zp = v.k_zp + (int64_t)h * d_pad;
  const int64_t* perm = v.k_perm + (int64_t)h * v.k_perm_head_stride;
  const int nwarp = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int hq = 0; hq < g; ++hq) {
    float part = 0.f;
    for (int c = threadIdx.x; c < d_pad; c += blockDim.x) {
      float qs = load_q(q, q_dtype, q_head0_off + hq * q_row_stride + perm[c]) * h2f(sc[c]);
      smem_qs[hq * d_pad + c] = qs;
      part += h2f(zp[c]) * qs;
    }
    part = warp_sum(part);
    if (lane == 0) smem_red[warp * g + hq] = part;
  }
  __syncthreads();
  if (threadIdx.x < g) {
    float b = 0.f;
    for (int w = 0; w < nwarp; ++w) b += smem_red[w * g + threadIdx.x];
    smem_bias[threadIdx.x] = b;
  }
  __syncthreads();
}

// Raw code dot products of one stripe row against qs for heads [hq0, hq0+np).
__device__ __forceinline__ void row_dot(const rdkv_layer_view& v, int h, int64_t t, int d_pad,
                                        const float* smem_qs, int hq0, int np, float* acc) {
  const int sub2 = v.n_ch2_pad >> 2, sub4 = v.n_ch4_pad >> 1, n8 = v.n_ch8;
#pragma unroll
  for (int i = 0; i < GP; ++i) acc[i] = 0.f;
  if (sub2 > 0) {
    const uint8_t* row = v.k2 + h * v.k2_head_stride + t * sub2;
    for (int i = 0; i < sub2; ++i) {
      const unsigned b = row[i];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float code = (float)((b >> (2 * k)) & 3u);
        const float* qcol = smem_qs + hq0 * d_pad + i + k * sub2;
#pragma unroll
        for (int j = 0; j < GP; ++j)
          if (j < np) acc[j] = fmaf(code, qcol[j * d_pad], acc[j]);
      }
    }
  }
  if (sub4 > 0) {
    const uint8_t* row = v.k4 + h * v.k4_head_stride + t * sub4;
    const int base = v.n_ch2_pad;
    for (int i = 0; i < sub4; ++i) {
      const unsigned b = row[i];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const float code = (float)((b >> (4 * k)) & 15u);
        const float* qcol = smem_qs + hq0 * d_pad + base + i + k * sub4;
#pragma unroll
        for (int j = 0; j < GP; ++j)
          if (j < np) acc[j] = fmaf(code, qcol[j * d_pad], acc[j]);
      }
    }
  }
  if (n8 > 0) {
    const uint8_t* row = v.k8 + h * v.k8_head_stride + t * n8;
    const int base = v.n_ch2_pad + v.n_ch4_pad;
    for (int i = 0; i < n8; ++i) {
      const float code = (float)row[i];
      const float* qcol = smem_qs + hq0 * d_pad + base + i;
#pragma unroll
      for (int j = 0; j < GP; ++j)
        if (j < np) acc[j] = fmaf(code, qcol[j * d_pad], acc[j]);
    }
  }
}

// ───────────────────────────── K-side scores ────────────────────────────────
__global__ void __launch_bounds__(SCORE_THREADS)
k_scores_kernel(rdkv_layer_view v, const void* q, int q_dtype, int64_t q_row_stride, int g,
                int t_eff, float* out, int64_t out_row_stride) {
  extern __shared__ float smem[];
  const int h = blockIdx.y;
  const int d_pad = v.n_ch2_pad + v.n_ch4_pad + v.n_ch8;
  float* qs = smem;
  float* bias = qs + g * d_pad;
  float* red = bias + MAX_GROUP;
  setup_q(v, h, g, d_pad, q, q_dtype, (int64_t)h * g * q_row_stride, q_row_stride, qs, bias, red);
  const int64_t t = (int64_t)blockIdx.x * SCORE_THREADS + threadIdx.x;
  if (t >= t_eff) return;
  for (int hq0 = 0; hq0 < g; hq0 += GP) {
    const int np = min(GP, g - hq0);
    float acc[GP];
    row_dot(v, h, t, d_pad, qs, hq0, np, acc);
#pragma unroll
    for (int j = 0; j < GP; ++j)
      if (j < np) out[(int64_t)(h * g + hq0 + j) * out_row_stride + t] = (acc[j] - bias[hq0 + j]) * INV_SQRT_D;
  }
}

// ───────────────────── V rows: lane owns channels lane+32k ───────────────────
// kind: 0 = 2-bit row (32 B), 1 = 4-bit row (64 B), 2 = 8-bit row (128 B), 3 = fp16 row.
__device__ __forceinline__ void load_v_row(const rdkv_layer_view& v, int h, int kind, int64_t r,
                                           int lane, float* c) {
  if (kind == 0) {
    const unsigned b = v.v2[h * v.v2_head_stride + r * 32 + lane];
    c[0] = (float)(b & 3u); c[1] = (float)((b >> 2) & 3u);
    c[2] = (float)((b >> 4) & 3u); c[3] = (float)(b >> 6);
  } else if (kind == 1) {
    const uint8_t* row = v.v4 + h * v.v4_head_stride + r * 64;
    const unsigned b0 = row[lane], b1 = row[lane + 32];
    c[0] = (float)(b0 & 15u); c[2] = (float)(b0 >> 4);
    c[1] = (float)(b1 & 15u); c[3] = (float)(b1 >> 4);
  } else if (kind == 2) {
    const uint8_t* row = v.v8 + h * v.v8_head_stride + r * 128;
    c[0] = (float)row[lane]; c[1] = (float)row[lane + 32];
    c[2] = (float)row[lane + 64]; c[3] = (float)row[lane + 96];
  } else {
    const uint16_t* row = v.v16 + h * v.v16_head_stride + r * 128;
    c[0] = h2f(row[lane]); c[1] = h2f(row[lane + 32]);
    c[2] = h2f(row[lane + 64]); c[3] = h2f(row[lane + 96]);
  }
}

// Maps a head-local Zone-A row to its segment.  Returns kind and the row inside it.
__device__ __forceinline__ int zone_a_kind(const HeadCounts& hc, int r, int64_t* seg_row) {
  if (r < hc.n2) { *seg_row = r; return 0; }
  if (r < hc.n2 + hc.n4) { *seg_row = r - hc.n2; return 1; }
  *seg_row = r - hc.n2 - hc.n4; return 2;
}

// ─────────────────────────── V-side weighted sum ────────────────────────────
constexpr int VSUM_THREADS = 512;

__global__ void __launch_bounds__(VSUM_THREADS)
v_weighted_sum_kernel(rdkv_layer_view v, const float* w, int64_t w_row_stride, int g, float* out,
                      int64_t out_row_stride) {
  extern __shared__ float smem[];     // [nwarp][GP][128]
  const int h = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = VSUM_THREADS / 32;
  const HeadCounts hc = head_counts(v, h);
  const int rows = hc.t_v + hc.n16;
  for (int hq0 = 0; hq0 < g; hq0 += GP) {
    const int np = min(GP, g - hq0);
    float acc[GP][4];
#pragma unroll
    for (int j = 0; j < GP; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for (int r = warp; r < rows; r += nwarp) {
      float c[4];
      float sc = 1.f, zp = 0.f;
      int64_t col;
      if (r < hc.t_v) {
        int64_t seg_row;
        const int kind = zone_a_kind(hc, r, &seg_row);
        load_v_row(v, h, kind, seg_row, lane, c);
        sc = h2f(v.v_scale[h * v.v_meta_head_stride + r]);
        zp = h2f(v.v_zp[h * v.v_meta_head_stride + r]);
        col = r;
      } else {
        load_v_row(v, h, 3, r - hc.t_v, lane, c);
        col = (int64_t)v.max_t_v + (r - hc.t_v);
      }
#pragma unroll
      for (int j = 0; j < GP; ++j) {
        if (j < np) {
          const float ws = w[(int64_t)(h * g + hq0 + j) * w_row_stride + col] * sc;
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[j][k] = fmaf(ws, c[k] - zp, acc[j][k]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < GP; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) smem[(warp * GP + j) * D + lane + 32 * k] = acc[j][k];
    __syncthreads();
    for (int i = threadIdx.x; i < np * D; i += VSUM_THREADS) {
      const int j = i / D, d = i % D;
      float s = 0.f;
      for (int ww = 0; ww < nwarp; ++ww) s += smem[(ww * GP + j) * D + d];
      out[(int64_t)(h * g + hq0 + j) * out_row_stride + d] = s;
    }
    __syncthreads();
  }
}

// ───────────────────────────── LSE combine ───────────────────────────────────
__global__ void __launch_bounds__(D)
lse_combine_kernel(const float* __restrict__ partials, int n_splits, int64_t row_stride,
                   int64_t split_stride, float* __restrict__ out, float* __restrict__ out_ml,
                   float* __restrict__ out_partial) {
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x;
  const float* base = partials + row * row_stride;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[s * split_stride]);
  float L = 0.f, o = 0.f;
  if (M != -INFINITY) {
    for (int s = 0; s < n_splits; ++s) {
      const float* rec = base + s * split_stride;
      const float m = rec[0];
      if (m == -INFINITY) continue;
      const float wgt = exp2f((m - M) * 1.4426950408889634f);
      L = fmaf(rec[1], wgt, L);
      o = fmaf(rec[4 + d], wgt, o);
    }
  }
  if (out != nullptr) out[row * D + d] = (L > 0.f) ? o / L : 0.f;
  if (out_ml != nullptr && d == 0) { out_ml[row * 2] = M; out_ml[row * 2 + 1] = L; }
  if (out_partial != nullptr) {
    float* rec = out_partial + row * RDKV_PARTIAL_STRIDE;
    rec[4 + d] = o;
    if (d == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
  }
}

// ───────────────────────────── Zone C: uncompressed tail ─────────────────────
// Decode-appended tokens kept as plain K / V rows (reference: the new-token buffer of
// obkv_accel/fast_decode.py:863-866 and its scores / weighted sum, :1719-1784).  One warp per
// query head walks the tail with an online softmax and writes an (m, l, o[128]) record that
// the log-sum-exp combine merges with the packed zones' record: one softmax over all zones.
constexpr int TAIL_WARPS = 4;

__device__ __forceinline__ float4 load_row4(const void* base, int dtype, int64_t elem_off) {
  if (dtype == RDKV_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem_off);
  const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + elem_off);
  if (dtype == RDKV_F16) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

__global__ void __launch_bounds__(TAIL_WARPS * 32)
tail_attn_partial_kernel(const void* __restrict__ q, int q_dtype, int64_t n_rows, int H_q, int g,
                         const void* __restrict__ new_k, const void* __restrict__ new_v, int kv_dtype,
                         int64_t kv_view_stride, int64_t kv_head_stride, int64_t kv_row_stride, int n_new,
                         const int32_t* __restrict__ n_new_per_view, int cap, float* __restrict__ partial) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * TAIL_WARPS + warp;    // (view, query head)
  if (row >= n_rows) return;
  const int64_t view = row / H_q;
  const int hq = (int)(row % H_q), h = hq / g;
  const int n = min(max(n_new_per_view != nullptr ? n_new_per_view[view] : n_new, 0), cap);   // never past the buffer
  float4 qv;
  qv.x = load_q(q, q_dtype, row * D + 4 * lane) * INV_SQRT_D; qv.y = load_q(q, q_dtype, row * D + 4 * lane + 1) * INV_SQRT_D;
  qv.z = load_q(q, q_dtype, row * D + 4 * lane + 2) * INV_SQRT_D; qv.w = load_q(q, q_dtype, row * D + 4 * lane + 3) * INV_SQRT_D;
  const int64_t base = view * kv_view_stride + h * kv_head_stride + 4 * lane;
  float m = -INFINITY, l = 0.f;
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int t = 0; t < n; ++t) {
    const float4 k = load_row4(new_k, kv_dtype, base + t * kv_row_stride);
    const float4 vv = load_row4(new_v, kv_dtype, base + t * kv_row_stride);
    float sdot = warp_sum(qv.x * k.x + qv.y * k.y + qv.z * k.z + qv.w * k.w);
    sdot = __shfl_sync(0xffffffffu, sdot, 0);               // the same value in every lane
    const float mn = fmaxf(m, sdot);
    const float a = m == -INFINITY ? 0.f : __expf(m - mn), pw = __expf(sdot - mn);
    l = fmaf(l, a, pw);
    o.x = fmaf(o.x, a, pw * vv.x); o.y = fmaf(o.y, a, pw * vv.y);
    o.z = fmaf(o.z, a, pw * vv.z); o.w = fmaf(o.w, a, pw * vv.w);
    m = mn;
  }
  float* rec = partial + row * RDKV_PARTIAL_STRIDE;
  *reinterpret_cast<float4*>(rec + 4 + 4 * lane) = o;
  if (lane == 0) { rec[0] = m; rec[1] = l; rec[2] = 0.f; rec[3] = 0.f; }
}

static int check_view_dims(int H_q, int H_kv) {
  if (H_q <= 0 || H_kv <= 0) return RDKV_ERR_BAD_ARG;
  if (H_q % H_kv != 0 || H_q / H_kv > MAX_GROUP) return RDKV_ERR_BAD_SHAPE;
  return RDKV_OK;
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int rdkv_k_scores(const rdkv_layer_view* view, const void* q, int q_dtype,
                             int64_t q_row_stride, int H_q, int H_kv, int t_eff, float* out,
                             int64_t out_row_stride, void* stream) {
  if (view == nullptr || q == nullptr || out == nullptr || t_eff < 0) return RDKV_ERR_BAD_ARG;
  if (q_dtype < RDKV_F16 || q_dtype > RDKV_F32) return RDKV_ERR_BAD_ARG;
  int st = check_view_dims(H_q, H_kv);
  if (st != RDKV_OK) return st;
  if (t_eff == 0) return RDKV_OK;
  const int g = H_q / H_kv;
  const int d_pad = view->n_ch2_pad + view->n_ch4_pad + view->n_ch8;
  if (d_pad <= 0 || d_pad > 3 * D || (view->n_ch2_pad & 3) || (view->n_ch4_pad & 1)) return RDKV_ERR_BAD_SHAPE;
  if (view->k_scale == nullptr || view->k_zp == nullptr || view->k_perm == nullptr) return RDKV_ERR_BAD_ARG;
  if ((view->n_ch2_pad && !view->k2) || (view->n_ch4_pad && !view->k4) || (view->n_ch8 && !view->k8))
    return RDKV_ERR_BAD_ARG;
  const size_t smem = sizeof(float) * ((size_t)g * d_pad + MAX_GROUP + (SCORE_THREADS / 32) * MAX_GROUP);
  dim3 grid((t_eff + SCORE_THREADS - 1) / SCORE_THREADS, H_kv);
  k_scores_kernel<<<grid, SCORE_THREADS, smem, (cudaStream_t)stream>>>(
      *view, q, q_dtype, q_row_stride, g, t_eff, out, out_row_stride);
  return launch_status();
}

extern "C" int rdkv_v_weighted_sum(const rdkv_layer_view* view, const float* w, int64_t w_row_stride,
                                   int H_q, int H_kv, float* out, int64_t out_row_stride,
                                   void* stream) {
  if (view == nullptr || w == nullptr || out == nullptr) return RDKV_ERR_BAD_ARG;
  int st = check_view_dims(H_q, H_kv);
  if (st != RDKV_OK) return st;
  if (view->v_scale == nullptr || view->v_zp == nullptr) return RDKV_ERR_BAD_ARG;
  const int g = H_q / H_kv;
  const size_t smem = sizeof(float) * (VSUM_THREADS / 32) * GP * D;
  // (per device, not per process: set on every call, as the fused kernel's launcher does)
  cudaError_t e = cudaFuncSetAttribute(v_weighted_sum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  v_weighted_sum_kernel<<<H_kv, VSUM_THREADS, smem, (cudaStream_t)stream>>>(*view, w, w_row_stride, g, out,
                                                                           out_row_stride);
  return launch_status();
}

extern "C" int rdkv_lse_combine(const float* partials, int64_t n_rows, int n_splits, int64_t row_stride,
                                int64_t split_stride, float* out, float* out_ml, float* out_partial,
                                void* stream) {
  if (partials == nullptr || n_rows < 0 || n_splits <= 0) return RDKV_ERR_BAD_ARG;
  if (out == nullptr && out_partial == nullptr) return RDKV_ERR_BAD_ARG;
  if (n_rows == 0) return RDKV_OK;
  if (n_rows > 0x7fffffffLL) return RDKV_ERR_TOO_LARGE;
  lse_combine_kernel<<<(unsigned)n_rows, D, 0, (cudaStream_t)stream>>>(partials, n_splits, row_stride,
                                                                      split_stride, out, out_ml,
                                                                      out_partial);
  return launch_status();
}

extern "C" int rdkv_tail_attn_partial(const void* q, int q_dtype, int64_t n_views, int H_q, int H_kv,
                                      const void* new_k, const void* new_v, int kv_dtype,
                                      int64_t kv_view_stride, int64_t kv_head_stride, int64_t kv_row_stride,
                                      int n_new, const int32_t* n_new_per_view, int cap, float* partial, void* stream) {
  if (q == nullptr || new_k == nullptr || new_v == nullptr || partial == nullptr || n_views < 0 || n_new < 0 ||
      cap < 0 || n_new > cap)
    return RDKV_ERR_BAD_ARG;
  if (q_dtype < RDKV_F16 || q_dtype > RDKV_F32 || kv_dtype < RDKV_F16 || kv_dtype > RDKV_F32) return RDKV_ERR_BAD_ARG;
  if (H_q <= 0 || H_kv <= 0 || H_q % H_kv != 0) return RDKV_ERR_BAD_SHAPE;
  const int align = kv_dtype == RDKV_F32 ? 4 : 4;            // rows are read 4 elements per lane
  if ((kv_view_stride % align) || (kv_head_stride % align) || (kv_row_stride % align)) return RDKV_ERR_BAD_SHAPE;
  const size_t bytes = kv_dtype == RDKV_F32 ? 16 : 8;
  if ((reinterpret_cast<uintptr_t>(new_k) % bytes) || (reinterpret_cast<uintptr_t>(new_v) % bytes) ||
      (reinterpret_cast<uintptr_t>(partial) % 16))
    return RDKV_ERR_BAD_ARG;
  const int64_t n_rows = n_views * H_q;
  if (n_rows == 0) return RDKV_OK;
  const int64_t blocks = (n_rows + TAIL_WARPS - 1) / TAIL_WARPS;
  if (blocks > 0x7fffffffLL) return RDKV_ERR_TOO_LARGE;
  tail_attn_partial_kernel<<<(unsigned)blocks, TAIL_WARPS * 32, 0, (cudaStream_t)stream>>>(
      q, q_dtype, n_rows, H_q, H_q / H_kv, new_k, new_v, kv_dtype, kv_view_stride, kv_head_stride, kv_row_stride,
      n_new, n_new_per_view, cap, partial);
  return launch_status();
}
