// Prefill quantise-and-bitpack: stable partition of the bit maps, per-token V
// packing and per-channel K packing on the stripe.
//
// Bit-exactness contract (reference: obkv_accel/packing.py:141-165): fp32 math
// with one IEEE rounding per operation — true division (__fdiv_rn), no fused
// multiply-add, round-half-to-even (rintf), fp16 outputs rounded to nearest.
#include "rdkv_common.cuh"

namespace rdkv {

// ───────────────────────────── partition by bits ─────────────────────────────
constexpr int PART_THREADS = 1024;

__device__ __forceinline__ int64_t load_int(const void* p, int elem_size, int64_t i) {
  switch (elem_size) {
    case 1: return reinterpret_cast<const int8_t*>(p)[i];
    case 2: return reinterpret_cast<const int16_t*>(p)[i];
    case 4: return reinterpret_cast<const int32_t*>(p)[i];
    default: return reinterpret_cast<const int64_t*>(p)[i];
  }
}

__device__ __forceinline__ int bit_class(int64_t b, int mode) {
  if (b == 2) return 0;
  if (b == 4) return 1;
  if (b == 8) return 2;
  if (b == 16) return mode == 0 ? 3 : 2;
  return -1;
}

__global__ void __launch_bounds__(PART_THREADS)
partition_kernel(const void* bits, int elem_size, int64_t row_stride, int len, int mode,
                 int32_t* order, int32_t* counts) {
  __shared__ int warp_tot[4][PART_THREADS / 32];
  __shared__ int class_base[5];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t off = (int64_t)row * row_stride;
  const int per = (len + PART_THREADS - 1) / PART_THREADS;
  const int lo = min(len, tid * per), hi = min(len, lo + per);
  int cnt[4] = {0, 0, 0, 0};
  for (int i = lo; i < hi; ++i) {
    const int c = bit_class(load_int(bits, elem_size, off + i), mode);
    if (c >= 0) cnt[c]++;
  }
  int excl[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    int v = cnt[c];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    excl[c] = v - cnt[c];
    if (lane == 31) warp_tot[c][warp] = v;
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int v = warp_tot[c][lane];
      const int own = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      warp_tot[c][lane] = v - own;
      if (lane == 31) class_base[c + 1] = v;       // class totals (converted to bases below)
    }
  }
  __syncthreads();
  if (tid == 0) {
    const int n0 = class_base[1], n1 = class_base[2], n2 = class_base[3], n3 = class_base[4];
    counts[row * 4 + 0] = n0; counts[row * 4 + 1] = n1; counts[row * 4 + 2] = n2; counts[row * 4 + 3] = n3;
    class_base[0] = 0; class_base[1] = n0; class_base[2] = n0 + n1; class_base[3] = n0 + n1 + n2;
    class_base[4] = n0 + n1 + n2 + n3;
  }
  __syncthreads();
  int pos[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) pos[c] = class_base[c] + warp_tot[c][warp] + excl[c];
  int32_t* orow = order + (int64_t)row * len;
  for (int i = lo; i < hi; ++i) {
    const int c = bit_class(load_int(bits, elem_size, off + i), mode);
    if (c >= 0) orow[pos[c]++] = i;
  }
  const int kept = class_base[4];
  for (int i = kept + tid; i < len; i += PART_THREADS) orow[i] = -1;
}

// ───────────────────────────── quantisation core ─────────────────────────────
struct QParam { float scale, zp, qmax; };

__device__ __forceinline__ QParam make_qparam(float lo, float hi, float qmax) {
  QParam p;
  p.qmax = qmax;
  p.scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), qmax), 1e-8f);
  p.zp = rintf(fminf(fmaxf(__fsub_rn(0.f, __fdiv_rn(lo, p.scale)), 0.f), qmax));
  return p;
}

__device__ __forceinline__ unsigned quant_code(float x, const QParam& p) {
  const float y = __fadd_rn(__fdiv_rn(x, p.scale), p.zp);
  return (unsigned)rintf(fminf(fmaxf(y, 0.f), p.qmax));
}

__device__ __forceinline__ uint16_t f2h_bits(float x) { return __half_as_ushort(__float2half_rn(x)); }

// ───────────────────────────── V: one warp per row ───────────────────────────
constexpr int PACKV_WARPS = 8;
constexpr int PACK_MAX_D = 512;

__global__ void __launch_bounds__(PACKV_WARPS * 32)
pack_v_kernel(const uint16_t* __restrict__ V, int64_t v_head_stride, int64_t v_row_stride, int D,
              const int32_t* __restrict__ order, int64_t order_row_stride,
              const int32_t* __restrict__ counts, int64_t counts_row_stride, int n_identity,
              int identity_bits, int max_n2, int max_n4, int max_n8, int max_n16,
              uint8_t* out2, uint8_t* out4, uint8_t* out8, uint16_t* out16, uint16_t* out_scale,
              uint16_t* out_zp, int max_t_v, int qbits_override) {
  __shared__ float xs[PACKV_WARPS][PACK_MAX_D];
  __shared__ uint8_t cs[PACKV_WARPS][PACK_MAX_D];
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int n[4];
  if (order != nullptr) {
    const int32_t* c = counts + h * counts_row_stride;
    n[0] = c[0]; n[1] = c[1]; n[2] = c[2]; n[3] = c[3];
  } else {
    n[0] = identity_bits == 2 ? n_identity : 0;
    n[1] = identity_bits == 4 ? n_identity : 0;
    n[2] = identity_bits == 8 ? n_identity : 0;
    n[3] = identity_bits == 16 ? n_identity : 0;
  }
  const int t_v = n[0] + n[1] + n[2];
  // zero the tail of the per-row metadata
  if (blockIdx.x == 0 && out_scale != nullptr) {
    for (int r = t_v + threadIdx.x; r < max_t_v; r += blockDim.x) {
      out_scale[(int64_t)h * max_t_v + r] = 0;
      out_zp[(int64_t)h * max_t_v + r] = 0;
    }
  }
  const int slots = max_n2 + max_n4 + max_n8 + max_n16;
  const int slot = blockIdx.x * PACKV_WARPS + warp;
  if (slot >= slots) return;
  int seg, j;
  if (slot < max_n2) { seg = 0; j = slot; }
  else if (slot < max_n2 + max_n4) { seg = 1; j = slot - max_n2; }
  else if (slot < max_n2 + max_n4 + max_n8) { seg = 2; j = slot - max_n2 - max_n4; }
  else { seg = 3; j = slot - max_n2 - max_n4 - max_n8; }
  const int base = seg == 0 ? 0 : seg == 1 ? n[0] : seg == 2 ? n[0] + n[1] : t_v;
  const bool live = j < n[seg];
  const int width = seg == 0 ? D / 4 : seg == 1 ? D / 2 : D;
  if (seg == 3) {                                   // fp16 rows are copied through
    uint16_t* dst = out16 + ((int64_t)h * max_n16 + j) * D;
    if (live) {
      const int src = order != nullptr ? order[h * order_row_stride + base + j] : j;
      const uint16_t* row = V + h * v_head_stride + (int64_t)src * v_row_stride;
      for (int c = lane; c < D; c += 32) dst[c] = row[c];
    } else {
      for (int c = lane; c < D; c += 32) dst[c] = 0;
    }
    return;
  }
  uint8_t* dst = seg == 0 ? out2 + ((int64_t)h * max_n2 + j) * width
               : seg == 1 ? out4 + ((int64_t)h * max_n4 + j) * width
                          : out8 + ((int64_t)h * max_n8 + j) * width;
  if (!live) {
    for (int c = lane; c < width; c += 32) dst[c] = 0;
    return;
  }
  const int src = order != nullptr ? order[h * order_row_stride + base + j] : j;
  const uint16_t* row = V + h * v_head_stride + (int64_t)src * v_row_stride;
  float lo = INFINITY, hi = -INFINITY;
  for (int c = lane; c < D; c += 32) {
    const float x = h2f(row[c]);
    xs[warp][c] = x;
    lo = fminf(lo, x); hi = fmaxf(hi, x);
  }
  lo = warp_min(lo); hi = warp_max(hi);
  const int qbits = qbits_override > 0 ? qbits_override : (seg == 0 ? 2 : seg == 1 ? 4 : 8);
  const QParam qp = make_qparam(lo, hi, (float)((1 << qbits) - 1));
  for (int c = lane; c < D; c += 32) cs[warp][c] = (uint8_t)quant_code(xs[warp][c], qp);
  __syncwarp();
  if (seg == 0) {
    const int S = D / 4;
    for (int i = lane; i < S; i += 32)
      dst[i] = cs[warp][i] | (cs[warp][i + S] << 2) | (cs[warp][i + 2 * S] << 4) | (cs[warp][i + 3 * S] << 6);
  } else if (seg == 1) {
    const int S = D / 2;
    for (int i = lane; i < S; i += 32) dst[i] = cs[warp][i] | (cs[warp][i + S] << 4);
  } else {
    for (int i = lane; i < D; i += 32) dst[i] = cs[warp][i];
  }
  if (lane == 0) {
    out_scale[(int64_t)h * max_t_v + base + j] = f2h_bits(qp.scale);
    out_zp[(int64_t)h * max_t_v + base + j] = f2h_bits(qp.zp);
  }
}

// ───────────────────────────── K: stripe maps ────────────────────────────────
struct KMaps {
  const int32_t* tok_order; int n2t, n4t, n8t, n16t;   // token partition of this head
  const int32_t* ch_order; int n2c, n4c, n8c;          // channel partition of this head
  int max_t_v, t_k, n2p, n4p, n8p;
};

__device__ __forceinline__ int stripe_token(const KMaps& m, int s) {
  if (m.tok_order == nullptr) return s;
  const int t_v = m.n2t + m.n4t + m.n8t;
  if (s < t_v) return m.tok_order[s];
  const int j = s - m.max_t_v;
  if (j >= 0 && j < m.n16t) return m.tok_order[t_v + j];
  return -1;
}

__device__ __forceinline__ int slot_channel(const KMaps& m, int p) {
  if (p < m.n2p) return p < m.n2c ? m.ch_order[p] : -1;
  p -= m.n2p;
  if (p < m.n4p) return p < m.n4c ? m.ch_order[m.n2c + p] : -1;
  p -= m.n4p;
  return p < m.n8c ? m.ch_order[m.n2c + m.n4c + p] : -1;
}

__device__ __forceinline__ KMaps load_maps(int h, const int32_t* tok_order, int64_t tok_order_rs,
                                           const int32_t* tok_counts, int64_t tok_counts_rs,
                                           int max_t_v, int t_k, const int32_t* ch_order,
                                           int64_t ch_order_rs, const int32_t* ch_counts,
                                           int64_t ch_counts_rs, int n2p, int n4p, int n8p) {
  KMaps m;
  m.tok_order = tok_order != nullptr ? tok_order + h * tok_order_rs : nullptr;
  if (tok_order != nullptr) {
    const int32_t* c = tok_counts + h * tok_counts_rs;
    m.n2t = c[0]; m.n4t = c[1]; m.n8t = c[2]; m.n16t = c[3];
  } else {
    m.n2t = m.n4t = m.n8t = m.n16t = 0;
  }
  m.ch_order = ch_order + h * ch_order_rs;
  const int32_t* cc = ch_counts + h * ch_counts_rs;
  m.n2c = cc[0]; m.n4c = cc[1]; m.n8c = cc[2];
  m.max_t_v = max_t_v; m.t_k = t_k; m.n2p = n2p; m.n4p = n4p; m.n8p = n8p;
  return m;
}

constexpr int PACKK_SLAB_ROWS = 64;
constexpr int PACKK_MAX_SLABS = 64;
constexpr int PACKK_MAX_DPAD = 3 * PACK_MAX_D;

__host__ __device__ inline int pack_k_slabs(int t_k) {
  int s = (t_k + PACKK_SLAB_ROWS - 1) / PACKK_SLAB_ROWS;
  return s < 1 ? 1 : (s > PACKK_MAX_SLABS ? PACKK_MAX_SLABS : s);
}

// Pass 1: per-slab min/max of every channel slot over its stripe rows.
__global__ void __launch_bounds__(128)
pack_k_minmax_kernel(const uint16_t* __restrict__ K, int64_t k_head_stride, int64_t k_row_stride,
                     const int32_t* tok_order, int64_t tok_order_rs, const int32_t* tok_counts,
                     int64_t tok_counts_rs, int max_t_v, int t_k, const int32_t* ch_order,
                     int64_t ch_order_rs, const int32_t* ch_counts, int64_t ch_counts_rs, int n2p,
                     int n4p, int n8p, float* __restrict__ scratch) {
  const int h = blockIdx.y, slab = blockIdx.x, n_slabs = gridDim.x;
  const KMaps m = load_maps(h, tok_order, tok_order_rs, tok_counts, tok_counts_rs, max_t_v, t_k,
                            ch_order, ch_order_rs, ch_counts, ch_counts_rs, n2p, n4p, n8p);
  const int d_pad = n2p + n4p + n8p;
  const int rows_per = (t_k + n_slabs - 1) / n_slabs;
  const int r0 = min(t_k, slab * rows_per), r1 = min(t_k, r0 + rows_per);
  for (int p = threadIdx.x; p < d_pad; p += blockDim.x) {
    const int ch = slot_channel(m, p);
    float lo = INFINITY, hi = -INFINITY;
    for (int s = r0; s < r1; ++s) {
      const int tok = stripe_token(m, s);
      const float x = (tok < 0 || ch < 0) ? 0.f : h2f(K[h * k_head_stride + (int64_t)tok * k_row_stride + ch]);
      lo = fminf(lo, x); hi = fmaxf(hi, x);
    }
    float* dst = scratch + ((int64_t)(h * n_slabs + slab) * 2) * d_pad;
    dst[p] = lo; dst[d_pad + p] = hi;
  }
}

// Pass 2: reduce slab extrema, quantise and bit-pack PACKK_ROWS stripe rows per CTA.
constexpr int PACKK_WARPS = 8;
constexpr int PACKK_ROWS = 32;

__global__ void __launch_bounds__(PACKK_WARPS * 32)
pack_k_quant_kernel(const uint16_t* __restrict__ K, int64_t k_head_stride, int64_t k_row_stride,
                    const int32_t* tok_order, int64_t tok_order_rs, const int32_t* tok_counts,
                    int64_t tok_counts_rs, int max_t_v, int t_k, const int32_t* ch_order,
                    int64_t ch_order_rs, const int32_t* ch_counts, int64_t ch_counts_rs, int n2p,
                    int n4p, int n8p, int d_kept_max, int gqa, int n_slabs,
                    const float* __restrict__ scratch, uint8_t* k2, uint8_t* k4, uint8_t* k8,
                    uint16_t* out_scale, uint16_t* out_zp, int64_t* sort_idx, int64_t* perm,
                    int64_t* perm_q, int32_t* seg_bounds, int qbits_override) {
  extern __shared__ unsigned char smem_raw[];
  const int d_pad = n2p + n4p + n8p;
  float* s_scale = reinterpret_cast<float*>(smem_raw);          // [d_pad]
  float* s_zp = s_scale + d_pad;                                 // [d_pad]
  int* s_ch = reinterpret_cast<int*>(s_zp + d_pad);             // [d_pad]
  uint8_t* s_codes = reinterpret_cast<uint8_t*>(s_ch + d_pad);  // [PACKK_WARPS][d_pad]
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const KMaps m = load_maps(h, tok_order, tok_order_rs, tok_counts, tok_counts_rs, max_t_v, t_k,
                            ch_order, ch_order_rs, ch_counts, ch_counts_rs, n2p, n4p, n8p);
  for (int p = threadIdx.x; p < d_pad; p += blockDim.x) {
    float lo = INFINITY, hi = -INFINITY;
    for (int s = 0; s < n_slabs; ++s) {
      const float* src = scratch + ((int64_t)(h * n_slabs + s) * 2) * d_pad;
      lo = fminf(lo, src[p]); hi = fmaxf(hi, src[d_pad + p]);
    }
    const int qbits = qbits_override > 0 ? qbits_override : (p < n2p ? 2 : p < n2p + n4p ? 4 : 8);
    const QParam qp = make_qparam(lo, hi, (float)((1 << qbits) - 1));
    s_scale[p] = qp.scale; s_zp[p] = qp.zp;
    const int ch = slot_channel(m, p);
    s_ch[p] = ch;
    if (blockIdx.x == 0) {
      out_scale[(int64_t)h * d_pad + p] = f2h_bits(qp.scale);
      out_zp[(int64_t)h * d_pad + p] = f2h_bits(qp.zp);
      const int64_t pc = ch < 0 ? 0 : ch;
      if (perm != nullptr) perm[(int64_t)h * d_pad + p] = pc;
      if (perm_q != nullptr)
        for (int i = 0; i < gqa; ++i) perm_q[((int64_t)h * gqa + i) * d_pad + p] = pc;
    }
  }
  if (blockIdx.x == 0) {
    const int kept = m.n2c + m.n4c + m.n8c;
    if (sort_idx != nullptr)
      for (int j = threadIdx.x; j < d_kept_max; j += blockDim.x)
        sort_idx[(int64_t)h * d_kept_max + j] = j < kept ? m.ch_order[j] : 0;
    if (seg_bounds != nullptr && threadIdx.x == 0) {
      seg_bounds[h * 3 + 0] = m.n2c; seg_bounds[h * 3 + 1] = m.n4c; seg_bounds[h * 3 + 2] = m.n8c;
    }
  }
  __syncthreads();
  const int sub2 = n2p / 4, sub4 = n4p / 2;
  uint8_t* codes = s_codes + warp * d_pad;
  const int row0 = blockIdx.x * PACKK_ROWS;
  for (int rr = warp; rr < PACKK_ROWS; rr += PACKK_WARPS) {
    const int s = row0 + rr;
    if (s >= t_k) break;
    const int tok = stripe_token(m, s);
    const uint16_t* row = K + h * k_head_stride + (int64_t)(tok < 0 ? 0 : tok) * k_row_stride;
    for (int p = lane; p < d_pad; p += 32) {
      const int ch = s_ch[p];
      const float x = (tok < 0 || ch < 0) ? 0.f : h2f(row[ch]);
      QParam qp;
      qp.scale = s_scale[p]; qp.zp = s_zp[p];
      qp.qmax = (float)((1 << (qbits_override > 0 ? qbits_override : (p < n2p ? 2 : p < n2p + n4p ? 4 : 8))) - 1);
      codes[p] = (uint8_t)quant_code(x, qp);
    }
    __syncwarp();
    if (qbits_override > 0) {
      for (int i = lane; i < d_pad; i += 32) k8[((int64_t)h * t_k + s) * d_pad + i] = codes[i];
    } else {
      for (int i = lane; i < sub2; i += 32)
        k2[((int64_t)h * t_k + s) * sub2 + i] =
            codes[i] | (codes[i + sub2] << 2) | (codes[i + 2 * sub2] << 4) | (codes[i + 3 * sub2] << 6);
      for (int i = lane; i < sub4; i += 32)
        k4[((int64_t)h * t_k + s) * sub4 + i] = codes[n2p + i] | (codes[n2p + i + sub4] << 4);
      for (int i = lane; i < n8p; i += 32) k8[((int64_t)h * t_k + s) * n8p + i] = codes[n2p + n4p + i];
    }
    __syncwarp();
  }
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int rdkv_partition_by_bits(const void* bits, int elem_size, int64_t row_stride, int n_rows,
                                      int len, int mode, int32_t* order, int32_t* counts, void* stream) {
  if (bits == nullptr || order == nullptr || counts == nullptr || n_rows < 0 || len < 0) return RDKV_ERR_BAD_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return RDKV_ERR_BAD_ARG;
  if (mode != 0 && mode != 1) return RDKV_ERR_BAD_ARG;
  if (n_rows == 0) return RDKV_OK;
  partition_kernel<<<n_rows, PART_THREADS, 0, (cudaStream_t)stream>>>(bits, elem_size, row_stride, len, mode,
                                                                     order, counts);
  return launch_status();
}

extern "C" int rdkv_pack_v(const uint16_t* V, int64_t v_head_stride, int64_t v_row_stride, int H, int D,
                           const int32_t* order, int64_t order_row_stride, const int32_t* counts,
                           int64_t counts_row_stride, int n_identity, int identity_bits, int max_n2,
                           int max_n4, int max_n8, int max_n16, uint8_t* out2, uint8_t* out4,
                           uint8_t* out8, uint16_t* out16, uint16_t* out_scale, uint16_t* out_zp,
                           int max_t_v, int quant_bits_override, void* stream) {
  if (V == nullptr || H <= 0 || D <= 0) return RDKV_ERR_BAD_ARG;
  if (D > PACK_MAX_D || (D & 3)) return RDKV_ERR_BAD_SHAPE;
  if (order != nullptr && counts == nullptr) return RDKV_ERR_BAD_ARG;
  if (max_n2 < 0 || max_n4 < 0 || max_n8 < 0 || max_n16 < 0 || max_t_v < 0) return RDKV_ERR_BAD_ARG;
  if ((max_n2 && !out2) || (max_n4 && !out4) || (max_n8 && !out8) || (max_n16 && !out16)) return RDKV_ERR_BAD_ARG;
  if (max_t_v > 0 && (out_scale == nullptr || out_zp == nullptr)) return RDKV_ERR_BAD_ARG;
  if (quant_bits_override < 0 || quant_bits_override > 8) return RDKV_ERR_BAD_ARG;
  const int slots = max_n2 + max_n4 + max_n8 + max_n16;
  if (slots == 0 && max_t_v == 0) return RDKV_OK;
  dim3 grid(slots > 0 ? (slots + PACKV_WARPS - 1) / PACKV_WARPS : 1, H);
  pack_v_kernel<<<grid, PACKV_WARPS * 32, 0, (cudaStream_t)stream>>>(
      V, v_head_stride, v_row_stride, D, order, order_row_stride, counts, counts_row_stride, n_identity,
      identity_bits, max_n2, max_n4, max_n8, max_n16, out2, out4, out8, out16, out_scale, out_zp,
      max_t_v, quant_bits_override);
  return launch_status();
}

extern "C" int rdkv_pack_k_slabs(int t_k) { return pack_k_slabs(t_k); }

extern "C" int rdkv_pack_k(const uint16_t* K, int64_t k_head_stride, int64_t k_row_stride, int H, int D,
                           const int32_t* tok_order, int64_t tok_order_row_stride,
                           const int32_t* tok_counts, int64_t tok_counts_row_stride, int max_t_v,
                           int t_k, const int32_t* ch_order, int64_t ch_order_row_stride,
                           const int32_t* ch_counts, int64_t ch_counts_row_stride, int n_ch2_pad,
                           int n_ch4_pad, int n_ch8, int d_kept_max, int gqa, float* scratch,
                           uint8_t* k2, uint8_t* k4, uint8_t* k8, uint16_t* out_scale, uint16_t* out_zp,
                           int64_t* sort_idx, int64_t* perm, int64_t* perm_q, int32_t* seg_bounds,
                           int quant_bits_override, void* stream) {
  if (K == nullptr || H <= 0 || D <= 0 || t_k <= 0 || scratch == nullptr) return RDKV_ERR_BAD_ARG;
  if (ch_order == nullptr || ch_counts == nullptr) return RDKV_ERR_BAD_ARG;
  if (tok_order != nullptr && tok_counts == nullptr) return RDKV_ERR_BAD_ARG;
  if (n_ch2_pad < 0 || n_ch4_pad < 0 || n_ch8 < 0 || (n_ch2_pad & 3) || (n_ch4_pad & 1)) return RDKV_ERR_BAD_SHAPE;
  const int d_pad = n_ch2_pad + n_ch4_pad + n_ch8;
  if (d_pad == 0) return RDKV_OK;
  if (d_pad > PACKK_MAX_DPAD) return RDKV_ERR_TOO_LARGE;
  if (out_scale == nullptr || out_zp == nullptr) return RDKV_ERR_BAD_ARG;
  if (quant_bits_override < 0 || quant_bits_override > 8) return RDKV_ERR_BAD_ARG;
  if (quant_bits_override > 0) {
    if (k8 == nullptr) return RDKV_ERR_BAD_ARG;
  } else if ((n_ch2_pad && !k2) || (n_ch4_pad && !k4) || (n_ch8 && !k8)) {
    return RDKV_ERR_BAD_ARG;
  }
  if (perm_q != nullptr && gqa <= 0) return RDKV_ERR_BAD_ARG;
  const int n_slabs = pack_k_slabs(t_k);
  cudaStream_t st = (cudaStream_t)stream;
  pack_k_minmax_kernel<<<dim3(n_slabs, H), 128, 0, st>>>(
      K, k_head_stride, k_row_stride, tok_order, tok_order_row_stride, tok_counts, tok_counts_row_stride,
      max_t_v, t_k, ch_order, ch_order_row_stride, ch_counts, ch_counts_row_stride, n_ch2_pad, n_ch4_pad,
      n_ch8, scratch);
  int rc = launch_status();
  if (rc != RDKV_OK) return rc;
  const size_t smem = (size_t)d_pad * (3 * sizeof(float)) + (size_t)PACKK_WARPS * d_pad;
  pack_k_quant_kernel<<<dim3((t_k + PACKK_ROWS - 1) / PACKK_ROWS, H), PACKK_WARPS * 32, smem, st>>>(
      K, k_head_stride, k_row_stride, tok_order, tok_order_row_stride, tok_counts, tok_counts_row_stride,
      max_t_v, t_k, ch_order, ch_order_row_stride, ch_counts, ch_counts_row_stride, n_ch2_pad, n_ch4_pad,
      n_ch8, d_kept_max, gqa, n_slabs, scratch, k2, k4, k8, out_scale, out_zp, sort_idx, perm, perm_q,
      seg_bounds, quant_bits_override);
  return launch_status();
}
