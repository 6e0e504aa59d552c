// Prefill quantise-and-bitpack: stable partition of the bit maps, per-token V
// packing and per-channel K packing on the stripe.
//
// Bit-exactness contract (reference: obkv_accel/packing.py:141-165): fp32 math
// with one IEEE rounding per operation — true division (__fdiv_rn), no fused
// multiply-add, round-half-to-even (rintf), fp16 outputs rounded to nearest.
#include <cooperative_groups.h>

#include <type_traits>

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
partition_kernel(const void* bits, int elem_size, int64_t row_stride, int len, int mode_flags,
                 int32_t* order, int32_t* counts) {
  const int mode = mode_flags & 1;                         // (bit 2 of mode_flags: leave the entries past the kept count alone)
  __shared__ int warp_tot[4][PART_THREADS / 32];
  __shared__ int class_base[5];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t off = (int64_t)row * row_stride;
  const int per = (len + PART_THREADS - 1) / PART_THREADS;
  const int lo = min(len, tid * per), hi = min(len, lo + per);
  int cnt[4] = {0, 0, 0, 0};
  // Up to 32 elements per thread are classified once and remembered as three bit masks (kept, class
  // bit 0, class bit 1), so the scatter pass below does not read the map again; 16-bit maps whose
  // per-thread chunks are 16-byte aligned are read with 16-byte loads.
  const bool cached = per <= 32;
  uint32_t m_keep = 0u, m_c0 = 0u, m_c1 = 0u;
  auto note = [&](int k, int64_t b) {
    const int c = bit_class(b, mode);
    if (c >= 0) {
      cnt[c]++;
      m_keep |= 1u << k; m_c0 |= (uint32_t)(c & 1) << k; m_c1 |= (uint32_t)(c >> 1) << k;
    }
  };
  const bool vec = cached && elem_size == 2 && (per & 7) == 0 && hi - lo == per &&
                   ((reinterpret_cast<uintptr_t>(bits) + 2 * (off + lo)) & 15) == 0;
  if (vec) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const int16_t*>(bits) + off + lo);
    uint4 w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) w[u] = u * 8 < per ? __ldg(src + u) : make_uint4(0u, 0u, 0u, 0u);
    // 16-bit values without branches: kept = a power of two in [2, 16]; class = log2 - 1 (16 counts as 8
    // for channel maps); the four class counts (at most 32 each) share one register, 8 bits apiece
    uint32_t cnt4 = 0u;
    auto note16 = [&](int k, uint32_t v) {
      const uint32_t ok = (uint32_t)((v - 2u <= 14u) & ((v & (v - 1u)) == 0u));
      uint32_t c = (30u - (uint32_t)__clz((int)(v | 1u))) & 3u;
      if (mode != 0) c = min(c, 2u);
      cnt4 += ok << (8u * c);
      m_keep |= ok << k; m_c0 |= (ok & c) << k; m_c1 |= (ok & (c >> 1)) << k;
    };
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (u * 8 >= per) break;
      const uint32_t x[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        note16(8 * u + 2 * e, x[e] & 0xFFFFu);
        note16(8 * u + 2 * e + 1, x[e] >> 16);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) cnt[c] = (int)((cnt4 >> (8 * c)) & 0xFFu);
  } else if (cached) {
    for (int i = lo; i < hi; ++i) note(i - lo, load_int(bits, elem_size, off + i));
  } else {
    for (int i = lo; i < hi; ++i) {
      const int c = bit_class(load_int(bits, elem_size, off + i), mode);
      if (c >= 0) cnt[c]++;
    }
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
  if (cached) {
    for (uint32_t m = m_keep; m != 0u; m &= m - 1) {       // kept elements in ascending order
      const int k = __ffs(m) - 1;
      const int c = ((m_c0 >> k) & 1u) | (((m_c1 >> k) & 1u) << 1);
      orow[pos[c]++] = lo + k;
    }
  } else {
    for (int i = lo; i < hi; ++i) {
      const int c = bit_class(load_int(bits, elem_size, off + i), mode);
      if (c >= 0) orow[pos[c]++] = i;
    }
  }
  if (mode_flags & 4) return;
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

// quant_code without the division in the common case.  rinv = RN(1/scale).  x*rinv differs from the
// rounded quotient by less than 2^-14.5 wherever the code is not decided by the clamp (|quotient| <= 256
// there: 2^-15 from the product, 2^-16 from the quotient's own rounding), so after adding the zero
// point (2^-17 per sum) the two sums differ by < 6.2e-5 and round to the same integer unless the
// sum lies within 1.3e-4 of a half-integer; those cases take the exact path.
// Non-finite inputs behave as in quant_code (NaN -> code 0, +-inf -> the clamp).
// The code comes back as a float (an exact small integer), so that callers can assemble bytes
// with exact fp32 multiply-adds and convert once per pair of bytes.  A sum outside the clamp range
// is decided by the clamp on both paths (its error is far below its distance to the range unless
// it is within 1.3e-4 of an end, where both round to that end), so the test looks at the clamped sum.
__device__ __forceinline__ float quant_code_fast_f(float x, float rinv, const QParam& p) {
  const float y = __fmaf_rn(x, rinv, p.zp);                 // (one rounding fewer than the bound allows for)
  const float yc = fminf(fmaxf(y, 0.f), p.qmax);
  const float c = __fadd_rn(__fadd_rn(yc, 12582912.f), -12582912.f);   // round half to even for 0 <= yc < 2^22
  if (fabsf(__fsub_rn(yc, c)) > 0.5f - 1.3e-4f) return (float)quant_code(x, p);
  return c;
}
__device__ __forceinline__ unsigned quant_code_fast(float x, float rinv, const QParam& p) {
  return (unsigned)quant_code_fast_f(x, rinv, p);
}

// min / max over the 32 lanes of a full warp in one instruction each (NaN operands are ignored,
// as by fminf / fmaxf)
__device__ __forceinline__ float warp_min_redux(float v) {
  float r;
  asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float warp_max_redux(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

__device__ __forceinline__ uint16_t f2h_bits(float x) { return __half_as_ushort(__float2half_rn(x)); }

// ───────────────────────────── V: one warp per row ───────────────────────────
constexpr int PACKV_WARPS = 8;
constexpr int PACK_MAX_D = 512;

// Arguments of one V packing pass (one layer).  rows2..rows16 / rows_meta: rows allocated per
// head in the output tensors (>= max_n*, max_t_v: the outputs may be slices of taller tensors).
struct PackVArgs {
  const uint16_t* V; int64_t v_head_stride, v_row_stride; int D;
  const int32_t* order; int64_t order_row_stride;
  const int32_t* counts; int64_t counts_row_stride;
  int n_identity, identity_bits, max_n2, max_n4, max_n8, max_n16;
  int rows2, rows4, rows8, rows16, rows_meta;
  uint8_t *out2, *out4, *out8; uint16_t *out16, *out_scale, *out_zp;
  int max_t_v, qbits_override;
};

__device__ __forceinline__ void pack_v_body(const PackVArgs& A, int h, int block_x,
                                            float (*xs)[PACK_MAX_D], uint8_t (*cs)[PACK_MAX_D]) {
  const uint16_t* __restrict__ V = A.V;
  const int64_t v_head_stride = A.v_head_stride, v_row_stride = A.v_row_stride, order_row_stride = A.order_row_stride;
  const int64_t counts_row_stride = A.counts_row_stride;
  const int D = A.D, n_identity = A.n_identity, identity_bits = A.identity_bits;
  const int max_n2 = A.max_n2, max_n4 = A.max_n4, max_n8 = A.max_n8, max_n16 = A.max_n16, max_t_v = A.max_t_v;
  const int qbits_override = A.qbits_override;
  const int32_t* __restrict__ order = A.order;
  const int32_t* __restrict__ counts = A.counts;
  uint8_t *out2 = A.out2, *out4 = A.out4, *out8 = A.out8;
  uint16_t *out16 = A.out16, *out_scale = A.out_scale, *out_zp = A.out_zp;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
  if (block_x == 0 && out_scale != nullptr) {
    for (int r = t_v + threadIdx.x; r < max_t_v; r += blockDim.x) {
      out_scale[(int64_t)h * A.rows_meta + r] = 0;
      out_zp[(int64_t)h * A.rows_meta + r] = 0;
    }
  }
  const int slots = max_n2 + max_n4 + max_n8 + max_n16;
  const int slot = block_x * PACKV_WARPS + warp;
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
    uint16_t* dst = out16 + ((int64_t)h * A.rows16 + j) * D;
    if (live) {
      const int src = order != nullptr ? order[h * order_row_stride + base + j] : j;
      const uint16_t* row = V + h * v_head_stride + (int64_t)src * v_row_stride;
      for (int c = lane; c < D; c += 32) dst[c] = row[c];
    } else {
      for (int c = lane; c < D; c += 32) dst[c] = 0;
    }
    return;
  }
  uint8_t* dst = seg == 0 ? out2 + ((int64_t)h * A.rows2 + j) * width
               : seg == 1 ? out4 + ((int64_t)h * A.rows4 + j) * width
                          : out8 + ((int64_t)h * A.rows8 + j) * width;
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
    out_scale[(int64_t)h * A.rows_meta + base + j] = f2h_bits(qp.scale);
    out_zp[(int64_t)h * A.rows_meta + base + j] = f2h_bits(qp.zp);
  }
}

// D == 128: four lanes per slot, eight slots per warp, everything in registers.  Lane s of a
// slot's four loads channels 32i + 8s .. +7 (i = 0..3) as 16-byte words and quantises them into four
// "planes" of eight one-byte codes; the packed row is then a few shifts and ORs of whole planes:
//   2-bit (byte b = channels b, b+32, b+64, b+96):  bytes 8s..8s+7  = P0 | P1<<2 | P2<<4 | P3<<6
//   4-bit (byte b = channels b, b+64):              bytes 32i+8s..  = P[i] | P[i+2]<<4   (i = 0, 1)
//   8-bit:                                          bytes 32i+8s..  = P[i]
// so codes never move between lanes and every store is 8 bytes.  The per-row work (where the row
// comes from, its extrema, scale and zero point) is paid once per eight rows of a warp instruction.
constexpr int PACKV_CTA_ROWS128 = PACKV_WARPS * 8;           // slots per CTA

__device__ __forceinline__ void store8(uint8_t* dst, uint2 v, bool aligned) {
  if (aligned) { *reinterpret_cast<uint2*>(dst) = v; return; }
#pragma unroll
  for (int e = 0; e < 8; ++e) dst[e] = (uint8_t)((e < 4 ? v.x : v.y) >> (8 * (e & 3)));
}

__device__ __forceinline__ void pack_v_body128(const PackVArgs& A, int h, int block_x) {
  constexpr int D = 128;
  const int s = threadIdx.x & 3;
  int n[4];
  {
    const int32_t* c = A.counts + h * A.counts_row_stride;
    n[0] = c[0]; n[1] = c[1]; n[2] = c[2]; n[3] = c[3];
  }
  const int t_v = n[0] + n[1] + n[2];
  if (block_x == 0 && A.out_scale != nullptr) {               // zero the tail of the per-row metadata
    for (int r = t_v + threadIdx.x; r < A.max_t_v; r += blockDim.x) {
      A.out_scale[(int64_t)h * A.rows_meta + r] = 0;
      A.out_zp[(int64_t)h * A.rows_meta + r] = 0;
    }
  }
  const int slots = A.max_n2 + A.max_n4 + A.max_n8 + A.max_n16;
  const int slot = block_x * PACKV_CTA_ROWS128 + (threadIdx.x >> 2);
  const bool in_range = slot < slots;                         // (lanes of idle slots still join the shuffles)
  int sg, j;
  if (slot < A.max_n2) { sg = 0; j = slot; }
  else if (slot < A.max_n2 + A.max_n4) { sg = 1; j = slot - A.max_n2; }
  else if (slot < A.max_n2 + A.max_n4 + A.max_n8) { sg = 2; j = slot - A.max_n2 - A.max_n4; }
  else { sg = 3; j = slot - A.max_n2 - A.max_n4 - A.max_n8; }
  const int base = sg == 0 ? 0 : sg == 1 ? n[0] : sg == 2 ? n[0] + n[1] : t_v;
  int src = -1;                                               // source token; -1: pad row (written as zeros)
  if (in_range && j < n[sg]) src = A.order[h * A.order_row_stride + base + j];
  const bool in_al = (reinterpret_cast<uintptr_t>(A.V) & 15) == 0 && (A.v_head_stride & 7) == 0 && (A.v_row_stride & 7) == 0;
  uint4 w[4];
  if (src >= 0) {
    const uint16_t* row = A.V + h * A.v_head_stride + (int64_t)src * A.v_row_stride + 8 * s;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (in_al) {
        w[i] = *reinterpret_cast<const uint4*>(row + 32 * i);
      } else {                                                // rows off 16-byte boundaries: element by element
        const uint16_t* e = row + 32 * i;
        w[i] = make_uint4((uint32_t)e[0] | (uint32_t)e[1] << 16, (uint32_t)e[2] | (uint32_t)e[3] << 16,
                          (uint32_t)e[4] | (uint32_t)e[5] << 16, (uint32_t)e[6] | (uint32_t)e[7] << 16);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (sg == 3) {                                              // fp16 rows are copied through (zeros when dead)
    if (in_range) {
      uint16_t* dst = A.out16 + ((int64_t)h * A.rows16 + j) * D + 8 * s;
      const bool al = (reinterpret_cast<uintptr_t>(A.out16) & 15) == 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (al) {
          *reinterpret_cast<uint4*>(dst + 32 * i) = w[i];
        } else {
          const uint32_t q[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
          for (int e = 0; e < 8; ++e) dst[32 * i + e] = (uint16_t)(q[e >> 1] >> (16 * (e & 1)));
        }
      }
    }
  }
  // extrema of the row: exact in fp16, over this lane's 32 channels and then the slot's four lanes
  __half2 lo2, hi2;
  {
    const uint32_t q0[4] = {w[0].x, w[0].y, w[0].z, w[0].w};
    lo2 = hi2 = *reinterpret_cast<const __half2*>(&q0[0]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t q[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __half2 v = *reinterpret_cast<const __half2*>(&q[e]);
        lo2 = __hmin2(lo2, v); hi2 = __hmax2(hi2, v);
      }
    }
  }
  float lo = fminf(__low2float(lo2), __high2float(lo2)), hi = fmaxf(__low2float(hi2), __high2float(hi2));
  lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 1)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, 1));
  lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 2)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, 2));
  if (!in_range || sg == 3) return;
  const int width = sg == 0 ? D / 4 : sg == 1 ? D / 2 : D;
  uint8_t* out = sg == 0 ? A.out2 : sg == 1 ? A.out4 : A.out8;
  const int64_t rows_out = sg == 0 ? A.rows2 : sg == 1 ? A.rows4 : A.rows8;
  const bool al = (reinterpret_cast<uintptr_t>(out) & 7) == 0;
  uint8_t* dst = out + ((int64_t)h * rows_out + j) * width + 8 * s;
  uint2 P[4];
  if (src >= 0) {
    const QParam qp = make_qparam(lo, hi, sg == 0 ? 3.f : sg == 1 ? 15.f : 255.f);
    const float rinv = __frcp_rn(qp.scale);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t q[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
      uint32_t pr[4];                                         // two one-byte codes each, from one fp16 pair
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&q[e]));
        const float c0 = quant_code_fast_f(x.x, rinv, qp), c1 = quant_code_fast_f(x.y, rinv, qp);
        pr[e] = (uint32_t)__fmaf_rn(c1, 256.f, c0);           // exact: both codes are integers <= 255
      }
      P[i] = make_uint2(pr[0] | pr[1] << 16, pr[2] | pr[3] << 16);
    }
    if (s == 0) {
      A.out_scale[(int64_t)h * A.rows_meta + base + j] = f2h_bits(qp.scale);
      A.out_zp[(int64_t)h * A.rows_meta + base + j] = f2h_bits(qp.zp);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) P[i] = make_uint2(0u, 0u);
  }
  if (sg == 0) {
    store8(dst, make_uint2(P[0].x | P[1].x << 2 | P[2].x << 4 | P[3].x << 6,
                           P[0].y | P[1].y << 2 | P[2].y << 4 | P[3].y << 6), al);
  } else if (sg == 1) {
    store8(dst, make_uint2(P[0].x | P[2].x << 4, P[0].y | P[2].y << 4), al);
    store8(dst + 32, make_uint2(P[1].x | P[3].x << 4, P[1].y | P[3].y << 4), al);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) store8(dst + 32 * i, P[i], al);
  }
}

__host__ __device__ inline bool pack_v_fast(int D, int qbits_override, const void* order) {
  return D == 128 && qbits_override == 0 && order != nullptr;
}
__host__ __device__ inline int pack_v_blocks(int slots, bool fast) {
  const int per = fast ? PACKV_CTA_ROWS128 : PACKV_WARPS;
  return slots > 0 ? (slots + per - 1) / per : 1;
}

__global__ void __launch_bounds__(PACKV_WARPS * 32)
pack_v128_kernel(PackVArgs A) {
  pack_v_body128(A, blockIdx.y, blockIdx.x);
}

__global__ void __launch_bounds__(PACKV_WARPS * 32)
pack_v_kernel(PackVArgs A) {
  __shared__ float xs[PACKV_WARPS][PACK_MAX_D];
  __shared__ uint8_t cs[PACKV_WARPS][PACK_MAX_D];
  pack_v_body(A, blockIdx.y, blockIdx.x, xs, cs);
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

// Arguments of one K packing pass (one layer).  rows_k: stripe rows allocated per head in
// k2/k4/k8 (>= t_k: the outputs may be slices of taller tensors).
struct PackKArgs {
  const uint16_t* K; int64_t k_head_stride, k_row_stride;
  const int32_t* tok_order; int64_t tok_order_rs; const int32_t* tok_counts; int64_t tok_counts_rs;
  int max_t_v, t_k, rows_k;
  const int32_t* ch_order; int64_t ch_order_rs; const int32_t* ch_counts; int64_t ch_counts_rs;
  int n2p, n4p, n8p, d_kept_max, gqa, n_slabs;
  float* scratch;
  uint8_t *k2, *k4, *k8; uint16_t *out_scale, *out_zp;
  int64_t *sort_idx, *perm, *perm_q; int32_t* seg_bounds;
  int qbits_override;
  int stage_rows;                      // pass 3 reads whole 128-channel rows through shared memory
};

// Pass 1: per-slab min/max of every channel slot over its stripe rows.
__device__ __forceinline__ void pack_k_minmax_body(const PackKArgs& A, int h, int slab) {
  const uint16_t* __restrict__ K = A.K;
  const int64_t k_head_stride = A.k_head_stride, k_row_stride = A.k_row_stride;
  const int t_k = A.t_k, n2p = A.n2p, n4p = A.n4p, n8p = A.n8p, n_slabs = A.n_slabs;
  float* __restrict__ scratch = A.scratch;
  if (slab >= n_slabs) return;
  const KMaps m = load_maps(h, A.tok_order, A.tok_order_rs, A.tok_counts, A.tok_counts_rs, A.max_t_v, t_k,
                            A.ch_order, A.ch_order_rs, A.ch_counts, A.ch_counts_rs, n2p, n4p, n8p);
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
    float* dst = scratch + ((int64_t)(h * (n_slabs + 1) + slab) * 2) * d_pad;
    dst[p] = lo; dst[d_pad + p] = hi;
  }
}

// D == 128: the slab's rows are read whole (one 8-byte load per lane and row, several rows in
// flight per warp) and the extrema of ALL 128 channels are kept in registers; the kept channels
// are picked out at the end.  Rows without a token and slots without a channel count as zeros,
// as on the zero-padded canvas the reference quantises.
__device__ __forceinline__ void pack_k_minmax_body128(const PackKArgs& A, int h, int slab) {
  __shared__ float s_lo[4][128], s_hi[4][128];
  __shared__ int s_pad[4];
  const int t_k = A.t_k, n_slabs = A.n_slabs;
  if (slab >= n_slabs) return;
  const int n2p = A.n2p, n4p = A.n4p, n8p = A.n8p, d_pad = n2p + n4p + n8p;
  const KMaps m = load_maps(h, A.tok_order, A.tok_order_rs, A.tok_counts, A.tok_counts_rs, A.max_t_v, t_k,
                            A.ch_order, A.ch_order_rs, A.ch_counts, A.ch_counts_rs, n2p, n4p, n8p);
  const int rows_per = (t_k + n_slabs - 1) / n_slabs;
  const int r0 = min(t_k, slab * rows_per), r1 = min(t_k, r0 + rows_per);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // extrema in fp16 pairs (exact: the data are fp16), two pairs per lane = channels 4*lane .. +3;
  // the tokens of 16 stripe rows are looked up one per lane and handed round by shuffle, and the
  // 16 rows are loaded together
  const __half2 inf2 = __float2half2_rn(INFINITY), ninf2 = __float2half2_rn(-INFINITY);
  __half2 lo2[2] = {inf2, inf2}, hi2[2] = {ninf2, ninf2};
  bool pad = false;
  const uint16_t* Kh = A.K + h * A.k_head_stride + 4 * lane;
  for (int s0 = r0 + warp * 16; s0 < r1; s0 += 64) {          // 4 warps x 16 rows per round
    const int tok_l = (lane < 16 && s0 + lane < r1) ? stripe_token(m, s0 + lane) : -2;
    pad = pad || __any_sync(0xffffffffu, tok_l == -1);
    {
      uint2 w[16];
      bool on[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const int tok = __shfl_sync(0xffffffffu, tok_l, k);
        on[k] = tok >= 0;
        w[k] = make_uint2(0u, 0u);
        if (on[k]) w[k] = *reinterpret_cast<const uint2*>(Kh + (int64_t)tok * A.k_row_stride);
      }
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        if (!on[k]) continue;                                  // (warp-uniform)
        const __half2 a = *reinterpret_cast<const __half2*>(&w[k].x), c = *reinterpret_cast<const __half2*>(&w[k].y);
        lo2[0] = __hmin2(lo2[0], a); hi2[0] = __hmax2(hi2[0], a);
        lo2[1] = __hmin2(lo2[1], c); hi2[1] = __hmax2(hi2[1], c);
      }
    }
  }
  {
    const float2 l0 = __half22float2(lo2[0]), l1 = __half22float2(lo2[1]);
    const float2 h0 = __half22float2(hi2[0]), h1 = __half22float2(hi2[1]);
    s_lo[warp][4 * lane + 0] = l0.x; s_lo[warp][4 * lane + 1] = l0.y; s_lo[warp][4 * lane + 2] = l1.x; s_lo[warp][4 * lane + 3] = l1.y;
    s_hi[warp][4 * lane + 0] = h0.x; s_hi[warp][4 * lane + 1] = h0.y; s_hi[warp][4 * lane + 2] = h1.x; s_hi[warp][4 * lane + 3] = h1.y;
  }
  if (lane == 0) s_pad[warp] = pad ? 1 : 0;
  __syncthreads();
  const bool any_pad = (s_pad[0] | s_pad[1] | s_pad[2] | s_pad[3]) != 0;
  float* dst = A.scratch + ((int64_t)(h * (n_slabs + 1) + slab) * 2) * d_pad;
  for (int p = threadIdx.x; p < d_pad; p += blockDim.x) {
    const int ch = slot_channel(m, p);
    float l = INFINITY, u = -INFINITY;
    if (r1 > r0) {
      if (ch < 0) { l = 0.f; u = 0.f; }
      else {
        l = fminf(fminf(s_lo[0][ch], s_lo[1][ch]), fminf(s_lo[2][ch], s_lo[3][ch]));
        u = fmaxf(fmaxf(s_hi[0][ch], s_hi[1][ch]), fmaxf(s_hi[2][ch], s_hi[3][ch]));
        if (any_pad) { l = fminf(l, 0.f); u = fmaxf(u, 0.f); }
      }
    }
    dst[p] = l; dst[d_pad + p] = u;
  }
}

__host__ __device__ inline bool pack_k_fast(int D, int64_t k_row_stride, const void* K) {
  return D == 128 && (k_row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(K) & 7) == 0;
}

__global__ void __launch_bounds__(128)
pack_k_minmax_kernel(PackKArgs A) { pack_k_minmax_body(A, blockIdx.y, blockIdx.x); }

__global__ void __launch_bounds__(128)
pack_k_minmax128_kernel(PackKArgs A) { pack_k_minmax_body128(A, blockIdx.y, blockIdx.x); }

// Pass 2 (one CTA per head): reduce the slab extrema to scale / zero point per channel slot
// (kept in fp32 in the head's last scratch block for pass 3) and write the per-head tables.
__device__ __forceinline__ void pack_k_params_body(const PackKArgs& A, int h) {
  const int n2p = A.n2p, n4p = A.n4p, n8p = A.n8p, n_slabs = A.n_slabs, gqa = A.gqa;
  const int d_pad = n2p + n4p + n8p;
  const KMaps m = load_maps(h, A.tok_order, A.tok_order_rs, A.tok_counts, A.tok_counts_rs, A.max_t_v, A.t_k,
                            A.ch_order, A.ch_order_rs, A.ch_counts, A.ch_counts_rs, n2p, n4p, n8p);
  float* fin = A.scratch + ((int64_t)(h * (n_slabs + 1) + n_slabs) * 2) * d_pad;
  // narrow heads: the slabs of a slot are reduced by PARAM_PARTS threads side by side first
  constexpr int PARAM_PARTS = 8, PARAM_DMAX = 128;
  __shared__ float s_part[2][PARAM_PARTS][PARAM_DMAX];
  const bool split = d_pad <= PARAM_DMAX;
  if (split) {
    for (int idx = threadIdx.x; idx < d_pad * PARAM_PARTS; idx += blockDim.x) {
      const int p = idx % d_pad, part = idx / d_pad;
      float lo = INFINITY, hi = -INFINITY;
      for (int s = part; s < n_slabs; s += PARAM_PARTS) {
        const float* src = A.scratch + ((int64_t)(h * (n_slabs + 1) + s) * 2) * d_pad;
        lo = fminf(lo, src[p]); hi = fmaxf(hi, src[d_pad + p]);
      }
      s_part[0][part][p] = lo; s_part[1][part][p] = hi;
    }
    __syncthreads();
  }
  for (int p = threadIdx.x; p < d_pad; p += blockDim.x) {
    float lo = INFINITY, hi = -INFINITY;
    if (split) {
#pragma unroll
      for (int part = 0; part < PARAM_PARTS; ++part) {
        lo = fminf(lo, s_part[0][part][p]); hi = fmaxf(hi, s_part[1][part][p]);
      }
    } else {
      for (int s = 0; s < n_slabs; ++s) {
        const float* src = A.scratch + ((int64_t)(h * (n_slabs + 1) + s) * 2) * d_pad;
        lo = fminf(lo, src[p]); hi = fmaxf(hi, src[d_pad + p]);
      }
    }
    const int qbits = A.qbits_override > 0 ? A.qbits_override : (p < n2p ? 2 : p < n2p + n4p ? 4 : 8);
    const QParam qp = make_qparam(lo, hi, (float)((1 << qbits) - 1));
    fin[p] = qp.scale; fin[d_pad + p] = qp.zp;
    A.out_scale[(int64_t)h * d_pad + p] = f2h_bits(qp.scale);
    A.out_zp[(int64_t)h * d_pad + p] = f2h_bits(qp.zp);
    const int ch = slot_channel(m, p);
    const int64_t pc = ch < 0 ? 0 : ch;
    if (A.perm != nullptr) A.perm[(int64_t)h * d_pad + p] = pc;
    if (A.perm_q != nullptr)
      for (int i = 0; i < gqa; ++i) A.perm_q[((int64_t)h * gqa + i) * d_pad + p] = pc;
  }
  const int kept = m.n2c + m.n4c + m.n8c;
  if (A.sort_idx != nullptr)
    for (int j = threadIdx.x; j < A.d_kept_max; j += blockDim.x)
      A.sort_idx[(int64_t)h * A.d_kept_max + j] = j < kept ? m.ch_order[j] : 0;
  if (A.seg_bounds != nullptr && threadIdx.x == 0) {
    A.seg_bounds[h * 3 + 0] = m.n2c; A.seg_bounds[h * 3 + 1] = m.n4c; A.seg_bounds[h * 3 + 2] = m.n8c;
  }
}

__global__ void __launch_bounds__(128)
pack_k_params_kernel(PackKArgs A) { pack_k_params_body(A, blockIdx.x); }

// Pass 3: quantise and bit-pack.  A CTA takes PACKK_BPC consecutive blocks of PACKK_ROWS stripe rows,
// so the per-head set-up (channel parameters, stripe-row -> token map) is paid once for all of
// them; each warp stages its own rows of the next block with cp.async while it quantises the
// current one (two buffers, no CTA-wide barrier in the loop).
constexpr int PACKK_WARPS = 8;
constexpr int PACKK_ROWS = 128;                              // stripe rows per block
constexpr int PACKK_RPW = PACKK_ROWS / PACKK_WARPS;          // rows per warp and block
constexpr int PACKK_BPC = 4;                                 // blocks per CTA

__host__ __device__ inline int pack_k_quant_ctas(int t_k) {
  return (t_k + PACKK_ROWS * PACKK_BPC - 1) / (PACKK_ROWS * PACKK_BPC);
}
__host__ __device__ inline size_t pack_k_quant_smem(int d_pad, bool staged) {
  return (size_t)d_pad * (3 * sizeof(float)) + (staged ? 16 + 2 * PACKK_ROWS * 128 * sizeof(uint16_t) : 0);
}

__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;"
               :: "r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// Dynamic shared memory: scale, zp (fp32) and channel (int) per slot, then — when rows are staged
// (128 channels, 8-byte aligned rows) — two buffers of PACKK_ROWS whole rows.
__device__ __forceinline__ void pack_k_quant_body(const PackKArgs& A, int h, int block_x, unsigned char* smem_raw) {
  __shared__ int s_tok[PACKK_ROWS * PACKK_BPC];
  const uint16_t* __restrict__ K = A.K;
  const int t_k = A.t_k, n2p = A.n2p, n4p = A.n4p, n8p = A.n8p, n_slabs = A.n_slabs, ov = A.qbits_override;
  const int64_t rows_k = A.rows_k;
  const int row_base = block_x * PACKK_ROWS * PACKK_BPC;
  if (row_base >= t_k) return;
  const int n_blocks = min(PACKK_BPC, (t_k - row_base + PACKK_ROWS - 1) / PACKK_ROWS);
  const int d_pad = n2p + n4p + n8p;
  float* s_scale = reinterpret_cast<float*>(smem_raw);          // [d_pad]
  float* s_zp = s_scale + d_pad;                                 // [d_pad]
  int* s_ch = reinterpret_cast<int*>(s_zp + d_pad);             // [d_pad]
  uint16_t* s_rows = reinterpret_cast<uint16_t*>(smem_raw + (((size_t)d_pad * 12 + 15) & ~(size_t)15));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const KMaps m = load_maps(h, A.tok_order, A.tok_order_rs, A.tok_counts, A.tok_counts_rs, A.max_t_v, t_k,
                            A.ch_order, A.ch_order_rs, A.ch_counts, A.ch_counts_rs, n2p, n4p, n8p);
  const float* fin = A.scratch + ((int64_t)(h * (n_slabs + 1) + n_slabs) * 2) * d_pad;
  for (int p = threadIdx.x; p < d_pad; p += blockDim.x) {
    s_scale[p] = fin[p]; s_zp[p] = fin[d_pad + p]; s_ch[p] = slot_channel(m, p);
  }
  for (int i = threadIdx.x; i < n_blocks * PACKK_ROWS; i += blockDim.x)
    s_tok[i] = row_base + i < t_k ? stripe_token(m, row_base + i) : -1;
  __syncthreads();
  const uint16_t* Kh = K + h * A.k_head_stride;
  const bool staged = A.stage_rows != 0;
  auto stage = [&](int blk) {                                  // this warp's rows of block blk -> buffer blk & 1
    uint16_t* buf = s_rows + (blk & 1) * PACKK_ROWS * 128;
#pragma unroll
    for (int k = 0; k < PACKK_RPW; ++k) {
      const int i = warp * PACKK_RPW + k;
      const int tok = s_tok[blk * PACKK_ROWS + i];
      uint16_t* dst = buf + i * 128 + 4 * lane;
      if (tok >= 0) cp_async8(dst, Kh + (int64_t)tok * A.k_row_stride + 4 * lane);
      else *reinterpret_cast<uint2*>(dst) = make_uint2(0u, 0u);
    }
    cp_async_commit();
  };
  if (staged) stage(0);
  // A lane owns a "quad" of a row: four channel slots whose codes land in one output byte (2-bit),
  // two adjacent bytes (4-bit) or four adjacent bytes (8-bit), so codes never move between lanes
  // and all lanes carry the same number of codes.  Slots that do not exist (odd tails) get a zero
  // reciprocal and zero point, which quantises to code 0.
  const int sub2 = n2p / 4, sub4 = n4p / 2;
  const int nq2 = ov > 0 ? 0 : sub2, nq4 = ov > 0 ? 0 : (sub4 + 1) / 2;
  const int n8 = ov > 0 ? d_pad : n8p, nq8 = (n8 + 3) / 4, base8 = ov > 0 ? 0 : n2p + n4p;
  // few quads per row (few kept channels): a warp works on 2 or 4 rows at once
  const int n_quads = nq2 + nq4 + nq8;
  const int qn = n_quads <= 8 ? 8 : n_quads <= 16 ? 16 : 32;   // lanes per row
  const int rpp = 32 / qn, rsub = lane / qn;                   // rows per pass, this lane's row of a pass
#pragma unroll 1
  for (int blk = 0; blk < n_blocks; ++blk) {
  if (staged) {
    if (blk + 1 < n_blocks) { stage(blk + 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncwarp();
  }
  const int row0 = row_base + blk * PACKK_ROWS;
  const uint16_t* rows_blk = s_rows + (blk & 1) * PACKK_ROWS * 128;
  for (int q = lane % qn; q < n_quads; q += qn) {
    int sl[4], nv, nb, shift, width, col;
    float qmax;
    uint8_t* dst;
    if (q < nq2) {
      nv = 4; nb = 1; shift = 2; qmax = 3.f; dst = A.k2; width = sub2; col = q;
#pragma unroll
      for (int v = 0; v < 4; ++v) sl[v] = q + v * sub2;
    } else if (q < nq2 + nq4) {
      const int b0 = 2 * (q - nq2);
      nb = b0 + 1 < sub4 ? 2 : 1; nv = 2 * nb; shift = 4; qmax = 15.f; dst = A.k4; width = sub4; col = b0;
      sl[0] = n2p + b0; sl[1] = n2p + b0 + sub4; sl[2] = n2p + b0 + 1; sl[3] = n2p + b0 + 1 + sub4;
    } else {
      const int b0 = 4 * (q - nq2 - nq4);
      nb = min(4, n8 - b0); nv = nb; shift = 8; qmax = ov > 0 ? (float)((1 << ov) - 1) : 255.f;
      dst = A.k8; width = n8; col = b0;
#pragma unroll
      for (int v = 0; v < 4; ++v) sl[v] = base8 + b0 + v;
    }
    int ch[4]; float sc[4], zp[4], rinv[4];
    bool live[4];                                              // the slot holds a kept channel
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const bool on = v < nv;
      const int x = on ? sl[v] : sl[0];
      ch[v] = s_ch[x]; sc[v] = s_scale[x];
      zp[v] = on ? s_zp[x] : 0.f;
      rinv[v] = on ? __frcp_rn(sc[v]) : 0.f;
      live[v] = ch[v] >= 0;
      ch[v] = max(ch[v], 0);
    }
    const float mult = (float)(1 << shift);
    uint8_t* out = dst + ((int64_t)h * rows_k + row0 + warp * PACKK_RPW) * width + col;
    // whole-word stores where every row's address allows it
    const int am = nb == 2 ? 1 : 3;
    const bool al = (nb == 2 || nb == 4) && (reinterpret_cast<uintptr_t>(out) & am) == 0 && (width & am) == 0;
    const int kmax = min(PACKK_RPW, t_k - row0 - warp * PACKK_RPW);     // rows of this warp that exist
    if (staged) {
      // shared-memory byte addresses of the four gathered elements in the warp's first row
      const uint32_t rw = (uint32_t)__cvta_generic_to_shared(rows_blk + warp * PACKK_RPW * 128);
      uint32_t ea[4];
#pragma unroll
      for (int v = 0; v < 4; ++v) ea[v] = rw + 2 * ch[v];
#pragma unroll 2
      for (int k = rsub; k < kmax; k += rpp) {
        float c[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint16_t bits;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(bits) : "r"(ea[v] + k * 256));
          const float x = live[v] ? h2f(bits) : 0.f;          // (staged rows of pad tokens were written as zeros)
          QParam qp; qp.scale = sc[v]; qp.zp = zp[v]; qp.qmax = qmax;
          c[v] = quant_code_fast_f(x, rinv[v], qp);
        }
        // codes are small integers: bytes assemble exactly in fp32 (at most 16 bits per half)
        const unsigned word = (unsigned)__fmaf_rn(c[1], mult, c[0]) | (unsigned)__fmaf_rn(c[3], mult, c[2]) << (2 * shift);
        uint8_t* o = out + (int64_t)k * width;
        if (nb == 1) o[0] = (uint8_t)word;
        else if (al && nb == 2) *reinterpret_cast<uint16_t*>(o) = (uint16_t)word;
        else if (al && nb == 4) *reinterpret_cast<uint32_t*>(o) = word;
        else {
          for (int e = 0; e < nb; ++e) o[e] = (uint8_t)(word >> (8 * e));
        }
      }
    } else {
#pragma unroll 2
      for (int k = rsub; k < kmax; k += rpp) {
        const int tok = s_tok[blk * PACKK_ROWS + warp * PACKK_RPW + k];
        const uint16_t* row = Kh + (int64_t)(tok < 0 ? 0 : tok) * A.k_row_stride;
        float c[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float x = (tok >= 0 && live[v]) ? h2f(row[ch[v]]) : 0.f;
          QParam qp; qp.scale = sc[v]; qp.zp = zp[v]; qp.qmax = qmax;
          c[v] = quant_code_fast_f(x, rinv[v], qp);
        }
        const unsigned word = (unsigned)__fmaf_rn(c[1], mult, c[0]) | (unsigned)__fmaf_rn(c[3], mult, c[2]) << (2 * shift);
        uint8_t* o = out + (int64_t)k * width;
        for (int e = 0; e < nb; ++e) o[e] = (uint8_t)(word >> (8 * e));
      }
    }
  }
  __syncwarp();                                                // the buffer may be restaged from here on
  }
}

__global__ void __launch_bounds__(PACKK_WARPS * 32)
pack_k_quant_kernel(PackKArgs A) {
  extern __shared__ __align__(16) unsigned char pk_smem[];
  pack_k_quant_body(A, blockIdx.y, blockIdx.x, pk_smem);
}

// ───────────────────────────── all layers in one launch ──────────────────────
// blockIdx.z = layer; the per-layer arguments come from a device array of jobs.
__device__ __forceinline__ void job_to_vargs(const rdkv_pack_job& J, PackVArgs& A) {
  A.V = J.V; A.v_head_stride = J.v_head_stride; A.v_row_stride = J.v_row_stride; A.D = J.D;
  A.order = J.tok_order; A.order_row_stride = J.tok_order_row_stride;
  A.counts = J.tok_counts; A.counts_row_stride = 4;
  A.n_identity = 0; A.identity_bits = 0;
  A.max_n2 = J.max_n2; A.max_n4 = J.max_n4; A.max_n8 = J.max_n8; A.max_n16 = J.max_n16;
  A.rows2 = J.rows2; A.rows4 = J.rows4; A.rows8 = J.rows8; A.rows16 = J.rows16; A.rows_meta = J.rows_meta;
  A.out2 = J.v2; A.out4 = J.v4; A.out8 = J.v8; A.out16 = J.v16; A.out_scale = J.v_scale; A.out_zp = J.v_zp;
  A.max_t_v = J.max_t_v; A.qbits_override = 0;
}

__global__ void __launch_bounds__(PACKV_WARPS * 32)
pack_v_batched_kernel(const rdkv_pack_job* __restrict__ jobs) {
  __shared__ float xs[PACKV_WARPS][PACK_MAX_D];
  __shared__ uint8_t cs[PACKV_WARPS][PACK_MAX_D];
  __shared__ PackVArgs A;
  if (threadIdx.x == 0) job_to_vargs(jobs[blockIdx.z], A);
  __syncthreads();
  pack_v_body(A, blockIdx.y, blockIdx.x, xs, cs);
}

__global__ void __launch_bounds__(PACKV_WARPS * 32)
pack_v128_batched_kernel(const rdkv_pack_job* __restrict__ jobs) {
  __shared__ PackVArgs A;
  if (threadIdx.x == 0) job_to_vargs(jobs[blockIdx.z], A);
  __syncthreads();
  pack_v_body128(A, blockIdx.y, blockIdx.x);
}

__device__ __forceinline__ void job_to_kargs(const rdkv_pack_job& J, PackKArgs& A) {
  A.K = J.K; A.k_head_stride = J.k_head_stride; A.k_row_stride = J.k_row_stride;
  A.tok_order = J.tok_order; A.tok_order_rs = J.tok_order_row_stride; A.tok_counts = J.tok_counts; A.tok_counts_rs = 4;
  A.max_t_v = J.max_t_v; A.t_k = J.t_k; A.rows_k = J.rows_k;
  A.ch_order = J.ch_order; A.ch_order_rs = J.ch_order_row_stride; A.ch_counts = J.ch_counts; A.ch_counts_rs = 4;
  A.n2p = J.n_ch2_pad; A.n4p = J.n_ch4_pad; A.n8p = J.n_ch8; A.d_kept_max = J.d_kept_max; A.gqa = J.gqa;
  A.n_slabs = pack_k_slabs(J.t_k); A.scratch = J.scratch;
  A.k2 = J.k2; A.k4 = J.k4; A.k8 = J.k8; A.out_scale = J.k_scale; A.out_zp = J.k_zp;
  A.sort_idx = J.sort_idx; A.perm = J.perm; A.perm_q = J.perm_q; A.seg_bounds = J.seg_bounds;
  A.qbits_override = 0;
  A.stage_rows = (pack_k_fast(J.D, J.k_row_stride, J.K) && (J.k_head_stride & 3) == 0) ? 1 : 0;
}

__global__ void __launch_bounds__(128)
pack_k_minmax_batched_kernel(const rdkv_pack_job* __restrict__ jobs) {
  __shared__ PackKArgs A;
  if (threadIdx.x == 0) job_to_kargs(jobs[blockIdx.z], A);
  __syncthreads();
  if (A.t_k <= 0 || A.n2p + A.n4p + A.n8p == 0) return;
  pack_k_minmax_body(A, blockIdx.y, blockIdx.x);
}

__global__ void __launch_bounds__(128)
pack_k_minmax128_batched_kernel(const rdkv_pack_job* __restrict__ jobs) {
  __shared__ PackKArgs A;
  if (threadIdx.x == 0) job_to_kargs(jobs[blockIdx.z], A);
  __syncthreads();
  if (A.t_k <= 0 || A.n2p + A.n4p + A.n8p == 0) return;
  if (pack_k_fast(128, A.k_row_stride, A.K + blockIdx.y * A.k_head_stride) && (A.k_head_stride & 3) == 0)
    pack_k_minmax_body128(A, blockIdx.y, blockIdx.x);
  else
    pack_k_minmax_body(A, blockIdx.y, blockIdx.x);
}

__global__ void __launch_bounds__(128)
pack_k_params_batched_kernel(const rdkv_pack_job* __restrict__ jobs) {
  __shared__ PackKArgs A;
  if (threadIdx.x == 0) job_to_kargs(jobs[blockIdx.y], A);
  __syncthreads();
  if (A.t_k <= 0 || A.n2p + A.n4p + A.n8p == 0) return;
  pack_k_params_body(A, blockIdx.x);
}

__global__ void __launch_bounds__(PACKK_WARPS * 32)
pack_k_quant_batched_kernel(const rdkv_pack_job* __restrict__ jobs) {
  extern __shared__ __align__(16) unsigned char pk_smem[];
  __shared__ PackKArgs A;
  if (threadIdx.x == 0) job_to_kargs(jobs[blockIdx.z], A);
  __syncthreads();
  if (A.t_k <= 0 || A.n2p + A.n4p + A.n8p == 0) return;
  pack_k_quant_body(A, blockIdx.y, blockIdx.x, pk_smem);
}

// ── K in ONE pass over the kept rows ─────────────────────────────────────────
// A thread-block cluster of KOP_CL CTAs per (layer, KV head); CTA c of the cluster owns the stripe
// rows [c*rows_per, (c+1)*rows_per).  Phase A: its warps gather those rows from the context (whole
// 256-byte rows, 16 in flight per warp), keep the extrema of all 128 channels in registers and park
// the KEPT channels of every row in shared memory (fp16, in the order the quantisation phase reads
// them: the four values of a lane's quad side by side).  The CTAs then publish
// their extrema per channel slot; after a cluster barrier every CTA reduces the eight sets (read
// from the other CTAs' shared memory; minima and maxima do not depend on the order) to scale and
// zero point per slot, and the first CTA writes the head's tables.  Phase B: every CTA quantises
// and bit-packs its own rows out of shared memory (the lane-quad scheme of pack_k_quant_body).
// The kept rows are read from DRAM once instead of twice.  128 channels, fp16 rows.
constexpr int KOP_CL = 8;
constexpr int KOP_WARPS = 8;
constexpr int KOP_MAX_SMEM = 200 * 1024;

__host__ __device__ inline int kop_rows_per_cta(int t_k) { return (((t_k + KOP_CL - 1) / KOP_CL) + 31) & ~31; }
// (a parked row holds a "quad" of four fp16 values per lane of the quantisation phase: at most
//  d_pad/4 + 2 quads of 8 bytes)
__host__ __device__ inline int kop_quads_bound(int d_pad) { return d_pad / 4 + 2; }
__host__ __device__ inline size_t kop_smem(int t_k, int d_pad, int quads) {
  return (size_t)d_pad * 20 + 256 + 16 + (size_t)kop_rows_per_cta(t_k) * 8 * quads;
}

__global__ void __launch_bounds__(KOP_WARPS * 32, 3)
pack_k_onepass_batched_kernel(const rdkv_pack_job* __restrict__ jobs, int rows_cap, int quads_cap) {
  namespace cg = cooperative_groups;
  extern __shared__ __align__(16) unsigned char kop_smem_raw[];
  __shared__ PackKArgs A;
  __shared__ __half2 s_wlo[KOP_WARPS][64], s_whi[KOP_WARPS][64];   // per warp: extrema of channel pairs
  __shared__ int s_pad[KOP_WARPS];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  if (threadIdx.x == 0) job_to_kargs(jobs[blockIdx.z], A);
  __syncthreads();
  const int t_k = A.t_k, n2p = A.n2p, n4p = A.n4p, n8p = A.n8p, d_pad = n2p + n4p + n8p;
  if (t_k <= 0 || d_pad == 0) return;                      // (the same for every CTA of the cluster)
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const KMaps m = load_maps(h, A.tok_order, A.tok_order_rs, A.tok_counts, A.tok_counts_rs, A.max_t_v, t_k,
                            A.ch_order, A.ch_order_rs, A.ch_counts, A.ch_counts_rs, n2p, n4p, n8p);
  float* s_ext = reinterpret_cast<float*>(kop_smem_raw);          // [2][d_pad] this CTA's extrema per slot
  float* s_scale = s_ext + 2 * d_pad;                              // [d_pad]
  float* s_zp = s_scale + d_pad;                                   // [d_pad]
  int* s_ch = reinterpret_cast<int*>(s_zp + d_pad);               // [d_pad] channel of a slot, or -1
  int16_t* s_c2s = reinterpret_cast<int16_t*>(s_ch + d_pad);      // [128] where a channel's value is parked in a row (fp16 index), or -1
  uint16_t* s_rows = reinterpret_cast<uint16_t*>(kop_smem_raw + (((size_t)d_pad * 20 + 256 + 15) & ~(size_t)15));
  const int rows_per = min(kop_rows_per_cta(t_k), rows_cap);
  const int r0 = min(t_k, rank * rows_per), r1 = min(t_k, r0 + rows_per), n_rows = r1 - r0;
  // quads of the quantisation phase: four channel slots whose codes land in one output byte (2-bit),
  // two adjacent bytes (4-bit) or four adjacent bytes (8-bit); slot p is value v of quad q
  const int sub2 = n2p / 4, sub4 = n4p / 2;
  const int nq2 = sub2, nq4 = (sub4 + 1) / 2, n8 = n8p, nq8 = (n8 + 3) / 4, base8 = n2p + n4p;
  const int n_quads = nq2 + nq4 + nq8;
  if (n_quads > quads_cap) return;                         // (the launch has no room for this layer's rows: refused on the host)
  const int row_h = 4 * n_quads;                                    // fp16 values per parked row
  auto park_pos = [&](int p) {
    if (p < n2p) return 4 * (p % sub2) + p / sub2;
    if (p < base8) { const int b = (p - n2p) % sub4, hi = (p - n2p) / sub4; return 4 * (nq2 + b / 2) + 2 * (b & 1) + hi; }
    return 4 * (nq2 + nq4) + (p - base8);
  };
  if (tid < 128) s_c2s[tid] = -1;
  {                                                         // rows start as zeros: slots without a channel, rows without a token
    uint4* z = reinterpret_cast<uint4*>(s_rows);
    const int n16 = (int)(((size_t)n_rows * row_h * 2 + 15) / 16);
    for (int i = tid; i < n16; i += blockDim.x) z[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  for (int p = tid; p < d_pad; p += blockDim.x) {
    const int ch = slot_channel(m, p);
    s_ch[p] = ch;
    if (ch >= 0) s_c2s[ch] = (int16_t)park_pos(p);
  }
  __syncthreads();

  // ── phase A: gather, extrema, kept channels to shared memory ──
  const bool aligned = pack_k_fast(128, A.k_row_stride, A.K + h * A.k_head_stride) && (A.k_head_stride & 3) == 0;
  int sl[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) sl[e] = s_c2s[4 * lane + e];
  const __half2 inf2 = __float2half2_rn(INFINITY), ninf2 = __float2half2_rn(-INFINITY);
  __half2 lo2[2] = {inf2, inf2}, hi2[2] = {ninf2, ninf2};
  bool pad = false;
  const uint16_t* Kh = A.K + h * A.k_head_stride + 4 * lane;
  // (shared-memory addresses as 32-bit offsets, the four parking places of this lane's channels as
  //  byte offsets within a row: the inner loop is a handful of instructions per row)
  const uint32_t rows32 = (uint32_t)__cvta_generic_to_shared(s_rows);
  const uint32_t rstride_b = 2u * (uint32_t)row_h;
  uint32_t off[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) off[e] = 2u * (uint32_t)max(sl[e], 0);
  const uint32_t kk0 = sl[0] >= 0, kk1 = sl[1] >= 0, kk2 = sl[2] >= 0, kk3 = sl[3] >= 0;
  const int64_t k_rs = A.k_row_stride;                     // (in registers: the loop below must not re-read A)
  auto gather = [&](auto AL) {
    constexpr bool ALIGNED = decltype(AL)::value;
    for (int s0 = r0 + warp * 16; s0 < r1; s0 += KOP_WARPS * 16) {
      const int tok_l = (lane < 16 && s0 + lane < r1) ? stripe_token(m, s0 + lane) : -2;
      pad = pad || __any_sync(0xffffffffu, tok_l == -1);
      uint2 w[16];
      int toks[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const int tok = __shfl_sync(0xffffffffu, tok_l, k);
        toks[k] = tok;
        w[k] = make_uint2(0u, 0u);
        if (tok >= 0) {
          const uint16_t* src = Kh + (int64_t)tok * k_rs;
          if (ALIGNED) w[k] = *reinterpret_cast<const uint2*>(src);
          else w[k] = make_uint2((uint32_t)src[0] | (uint32_t)src[1] << 16, (uint32_t)src[2] | (uint32_t)src[3] << 16);
        }
      }
      uint32_t rb = rows32 + (uint32_t)(s0 - r0) * rstride_b;
#pragma unroll
      for (int k = 0; k < 16; ++k, rb += rstride_b) {
        if (toks[k] < 0) continue;                           // (warp-uniform) no token: the row stays zeros
        const __half2 a = *reinterpret_cast<const __half2*>(&w[k].x), c = *reinterpret_cast<const __half2*>(&w[k].y);
        lo2[0] = __hmin2(lo2[0], a); hi2[0] = __hmax2(hi2[0], a);
        lo2[1] = __hmin2(lo2[1], c); hi2[1] = __hmax2(hi2[1], c);
        // predicated stores (no branches: the lanes of a warp differ in which channels they keep)
        asm volatile("{ .reg .pred p0, p1, p2, p3;\n"
                     ".reg .b16 a0, a1, a2, a3;\n"
                     "mov.b32 {a0, a1}, %4; mov.b32 {a2, a3}, %5;\n"
                     "setp.ne.u32 p0, %6, 0; setp.ne.u32 p1, %7, 0; setp.ne.u32 p2, %8, 0; setp.ne.u32 p3, %9, 0;\n"
                     "@p0 st.shared.u16 [%0], a0; @p1 st.shared.u16 [%1], a1;\n"
                     "@p2 st.shared.u16 [%2], a2; @p3 st.shared.u16 [%3], a3; }"
                     ::"r"(rb + off[0]), "r"(rb + off[1]), "r"(rb + off[2]), "r"(rb + off[3]), "r"(w[k].x), "r"(w[k].y),
                       "r"(kk0), "r"(kk1), "r"(kk2), "r"(kk3));
      }
    }
  };
  if (aligned) gather(std::true_type{}); else gather(std::false_type{});
  s_wlo[warp][2 * lane] = lo2[0]; s_wlo[warp][2 * lane + 1] = lo2[1];
  s_whi[warp][2 * lane] = hi2[0]; s_whi[warp][2 * lane + 1] = hi2[1];
  if (lane == 0) s_pad[warp] = pad ? 1 : 0;
  __syncthreads();
  {
    bool any_pad = false;
#pragma unroll
    for (int w = 0; w < KOP_WARPS; ++w) any_pad = any_pad || s_pad[w] != 0;
    for (int p = tid; p < d_pad; p += blockDim.x) {
      const int ch = s_ch[p];
      float l = INFINITY, u = -INFINITY;
      if (n_rows > 0) {
        if (ch < 0) { l = 0.f; u = 0.f; }
        else {
          const __half* wl = reinterpret_cast<const __half*>(&s_wlo[0][0]);
          const __half* wh = reinterpret_cast<const __half*>(&s_whi[0][0]);
#pragma unroll
          for (int w = 0; w < KOP_WARPS; ++w) {
            l = fminf(l, __half2float(wl[w * 128 + ch])); u = fmaxf(u, __half2float(wh[w * 128 + ch]));
          }
          if (any_pad) { l = fminf(l, 0.f); u = fmaxf(u, 0.f); }
        }
      }
      s_ext[p] = l; s_ext[d_pad + p] = u;
    }
  }
  cluster.sync();
  // ── the head's parameters from the eight CTAs' extrema ──
  for (int p = tid; p < d_pad; p += blockDim.x) {
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int rk = 0; rk < KOP_CL; ++rk) {
      const float* e = cluster.map_shared_rank(s_ext, rk);
      lo = fminf(lo, e[p]); hi = fmaxf(hi, e[d_pad + p]);
    }
    const int qbits = p < n2p ? 2 : p < n2p + n4p ? 4 : 8;
    const QParam qp = make_qparam(lo, hi, (float)((1 << qbits) - 1));
    s_scale[p] = qp.scale; s_zp[p] = qp.zp;
    if (rank == 0) {
      A.out_scale[(int64_t)h * d_pad + p] = f2h_bits(qp.scale);
      A.out_zp[(int64_t)h * d_pad + p] = f2h_bits(qp.zp);
      const int64_t pc = s_ch[p] < 0 ? 0 : s_ch[p];
      if (A.perm != nullptr) A.perm[(int64_t)h * d_pad + p] = pc;
      if (A.perm_q != nullptr)
        for (int i = 0; i < A.gqa; ++i) A.perm_q[((int64_t)h * A.gqa + i) * d_pad + p] = pc;
    }
  }
  if (rank == 0) {
    const int kept = m.n2c + m.n4c + m.n8c;
    if (A.sort_idx != nullptr)
      for (int j = tid; j < A.d_kept_max; j += blockDim.x)
        A.sort_idx[(int64_t)h * A.d_kept_max + j] = j < kept ? m.ch_order[j] : 0;
    if (A.seg_bounds != nullptr && tid == 0) {
      A.seg_bounds[h * 3 + 0] = m.n2c; A.seg_bounds[h * 3 + 1] = m.n4c; A.seg_bounds[h * 3 + 2] = m.n8c;
    }
  }
  cluster.sync();                                          // everybody has read everybody's extrema; parameters visible

  // ── phase B: quantise and bit-pack this CTA's rows out of shared memory ──
  const int64_t rows_k = A.rows_k;
  const int qn = n_quads <= 8 ? 8 : n_quads <= 16 ? 16 : 32;   // lanes per row
  const int rpp = 32 / qn, rsub = lane / qn;                   // rows per pass, this lane's row of a pass
  const int rpw = rows_per / KOP_WARPS;                        // rows per warp (a multiple of 4)
  const int wrow0 = warp * rpw;                                // this warp's first row within the CTA
  const int kmax = min(rpw, n_rows - wrow0);                   // rows of this warp that exist
  for (int q = lane % qn; q < n_quads; q += qn) {
    int slq[4], nv, nb, shift, width, col;
    float qmax;
    uint8_t* dst;
    if (q < nq2) {
      nv = 4; nb = 1; shift = 2; qmax = 3.f; dst = A.k2; width = sub2; col = q;
#pragma unroll
      for (int v = 0; v < 4; ++v) slq[v] = q + v * sub2;
    } else if (q < nq2 + nq4) {
      const int b0 = 2 * (q - nq2);
      nb = b0 + 1 < sub4 ? 2 : 1; nv = 2 * nb; shift = 4; qmax = 15.f; dst = A.k4; width = sub4; col = b0;
      slq[0] = n2p + b0; slq[1] = n2p + b0 + sub4; slq[2] = n2p + b0 + 1; slq[3] = n2p + b0 + 1 + sub4;
    } else {
      const int b0 = 4 * (q - nq2 - nq4);
      nb = min(4, n8 - b0); nv = nb; shift = 8; qmax = 255.f; dst = A.k8; width = n8; col = b0;
#pragma unroll
      for (int v = 0; v < 4; ++v) slq[v] = base8 + b0 + v;
    }
    float sc[4], zp[4], rinv[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const bool on = v < nv;
      const int x = on ? slq[v] : slq[0];
      sc[v] = s_scale[x];
      zp[v] = on ? s_zp[x] : 0.f;                            // (a value that does not exist is a parked zero: code 0)
      rinv[v] = on ? __frcp_rn(sc[v]) : 0.f;
    }
    const float mult = (float)(1 << shift);
    uint8_t* out = dst + ((int64_t)h * rows_k + r0 + wrow0) * width + col;
    const int am = nb == 2 ? 1 : 3;
    const bool al = (nb == 2 || nb == 4) && (reinterpret_cast<uintptr_t>(out) & am) == 0 && (width & am) == 0;
    const int how = nb == 1 ? 0 : (al && nb == 2) ? 1 : (al && nb == 4) ? 2 : 3;
    const uint32_t rstride = 2u * (uint32_t)row_h;
    const uint32_t qa = (uint32_t)__cvta_generic_to_shared(s_rows + (size_t)wrow0 * row_h) + 8u * (uint32_t)q;
#pragma unroll 2
    for (int k = rsub; k < kmax; k += rpp) {
      uint2 raw;                                             // the quad's four fp16 values of row k
      asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(raw.x), "=r"(raw.y) : "r"(qa + k * rstride));
      const float2 x01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
      const float2 x23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
      const float x[4] = {x01.x, x01.y, x23.x, x23.y};
      float c[4];
      bool tie = false;
#pragma unroll
      for (int v = 0; v < 4; ++v) {                          // quant_code_fast_f, the rare exact path taken for all four at once
        const float y = __fmaf_rn(x[v], rinv[v], zp[v]);
        const float yc = fminf(fmaxf(y, 0.f), qmax);
        c[v] = __fadd_rn(__fadd_rn(yc, 12582912.f), -12582912.f);
        tie = tie || fabsf(__fsub_rn(yc, c[v])) > 0.5f - 1.3e-4f;
      }
      if (tie) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          QParam qp; qp.scale = sc[v]; qp.zp = zp[v]; qp.qmax = qmax;
          c[v] = quant_code_fast_f(x[v], rinv[v], qp);
        }
      }
      // codes are small integers: bytes assemble exactly in fp32 (at most 16 bits per half)
      const unsigned word = (unsigned)__fmaf_rn(c[1], mult, c[0]) | (unsigned)__fmaf_rn(c[3], mult, c[2]) << (2 * shift);
      uint8_t* o = out + (int64_t)k * width;
      if (how == 0) o[0] = (uint8_t)word;
      else if (how == 1) *reinterpret_cast<uint16_t*>(o) = (uint16_t)word;
      else if (how == 2) *reinterpret_cast<uint32_t*>(o) = word;
      else {
        for (int e = 0; e < nb; ++e) o[e] = (uint8_t)(word >> (8 * e));
      }
    }
  }
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int rdkv_partition_by_bits(const void* bits, int elem_size, int64_t row_stride, int n_rows,
                                      int len, int mode, int32_t* order, int32_t* counts, void* stream) {
  if (bits == nullptr || order == nullptr || counts == nullptr || n_rows < 0 || len < 0) return RDKV_ERR_BAD_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return RDKV_ERR_BAD_ARG;
  if ((mode & ~4) != 0 && (mode & ~4) != 1) return RDKV_ERR_BAD_ARG;
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
  const bool fast = pack_v_fast(D, quant_bits_override, order);
  dim3 grid(pack_v_blocks(slots, fast), H);
  PackVArgs A;
  A.V = V; A.v_head_stride = v_head_stride; A.v_row_stride = v_row_stride; A.D = D;
  A.order = order; A.order_row_stride = order_row_stride; A.counts = counts; A.counts_row_stride = counts_row_stride;
  A.n_identity = n_identity; A.identity_bits = identity_bits;
  A.max_n2 = max_n2; A.max_n4 = max_n4; A.max_n8 = max_n8; A.max_n16 = max_n16;
  A.rows2 = max_n2; A.rows4 = max_n4; A.rows8 = max_n8; A.rows16 = max_n16; A.rows_meta = max_t_v;
  A.out2 = out2; A.out4 = out4; A.out8 = out8; A.out16 = out16; A.out_scale = out_scale; A.out_zp = out_zp;
  A.max_t_v = max_t_v; A.qbits_override = quant_bits_override;
  if (fast) pack_v128_kernel<<<grid, PACKV_WARPS * 32, 0, (cudaStream_t)stream>>>(A);
  else pack_v_kernel<<<grid, PACKV_WARPS * 32, 0, (cudaStream_t)stream>>>(A);
  return launch_status();
}

extern "C" int rdkv_pack_k_slabs(int t_k) { return pack_k_slabs(t_k) + 1; }

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
  PackKArgs A;
  A.K = K; A.k_head_stride = k_head_stride; A.k_row_stride = k_row_stride;
  A.tok_order = tok_order; A.tok_order_rs = tok_order_row_stride; A.tok_counts = tok_counts; A.tok_counts_rs = tok_counts_row_stride;
  A.max_t_v = max_t_v; A.t_k = t_k; A.rows_k = t_k;
  A.ch_order = ch_order; A.ch_order_rs = ch_order_row_stride; A.ch_counts = ch_counts; A.ch_counts_rs = ch_counts_row_stride;
  A.n2p = n_ch2_pad; A.n4p = n_ch4_pad; A.n8p = n_ch8; A.d_kept_max = d_kept_max; A.gqa = gqa; A.n_slabs = n_slabs;
  A.scratch = scratch; A.k2 = k2; A.k4 = k4; A.k8 = k8; A.out_scale = out_scale; A.out_zp = out_zp;
  A.sort_idx = sort_idx; A.perm = perm; A.perm_q = perm_q; A.seg_bounds = seg_bounds; A.qbits_override = quant_bits_override;
  A.stage_rows = (pack_k_fast(D, k_row_stride, K) && (k_head_stride & 3) == 0) ? 1 : 0;
  if (pack_k_fast(D, k_row_stride, K) && (k_head_stride & 3) == 0)
    pack_k_minmax128_kernel<<<dim3(n_slabs, H), 128, 0, st>>>(A);
  else
    pack_k_minmax_kernel<<<dim3(n_slabs, H), 128, 0, st>>>(A);
  int rc = launch_status();
  if (rc != RDKV_OK) return rc;
  pack_k_params_kernel<<<H, 128, 0, st>>>(A);
  rc = launch_status();
  if (rc != RDKV_OK) return rc;
  const size_t smem = pack_k_quant_smem(d_pad, A.stage_rows != 0);
  if (cudaFuncSetAttribute(pack_k_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return launch_status();
  pack_k_quant_kernel<<<dim3(pack_k_quant_ctas(t_k), H), PACKK_WARPS * 32, smem, st>>>(A);
  return launch_status();
}

extern "C" int rdkv_sizeof_pack_job(void) { return (int)sizeof(rdkv_pack_job); }

extern "C" int rdkv_pack_kv_batched(const rdkv_pack_job* jobs, int n_jobs, int H, int D, int max_slots,
                                    int max_t_k, int max_d_pad, int k_passes, int max_k_quads, void* stream) {
  if (k_passes != 0 && k_passes != 1 && k_passes != 3) return RDKV_ERR_BAD_ARG;
  if (max_k_quads < 0 || max_k_quads > kop_quads_bound(max_d_pad)) return RDKV_ERR_BAD_ARG;
  if (jobs == nullptr || n_jobs < 0 || H <= 0 || D <= 0 || max_slots < 0 || max_t_k < 0 || max_d_pad < 0)
    return RDKV_ERR_BAD_ARG;
  if (D > PACK_MAX_D || (D & 3)) return RDKV_ERR_BAD_SHAPE;
  if (max_d_pad > PACKK_MAX_DPAD) return RDKV_ERR_TOO_LARGE;
  if (n_jobs == 0) return RDKV_OK;
  if (n_jobs > 65535 || H > 65535) return RDKV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const bool fast = D == 128;
  dim3 gv(pack_v_blocks(max_slots, fast), H, n_jobs);
  if (fast) pack_v128_batched_kernel<<<gv, PACKV_WARPS * 32, 0, st>>>(jobs);
  else pack_v_batched_kernel<<<gv, PACKV_WARPS * 32, 0, st>>>(jobs);
  int rc = launch_status();
  if (rc != RDKV_OK || max_t_k == 0 || max_d_pad == 0) return rc;
  // K in one pass (the kept rows of a head held in the shared memory of a cluster) where they fit
  const int quads = max_k_quads > 0 ? max_k_quads : kop_quads_bound(max_d_pad);
  const size_t one_smem = kop_smem(max_t_k, max_d_pad, quads);
  const bool one_fits = D == 128 && one_smem <= (size_t)KOP_MAX_SMEM;
  if (k_passes == 1 && !one_fits) return RDKV_ERR_TOO_LARGE;
  if (one_fits && k_passes != 3) {
    cudaError_t e = cudaFuncSetAttribute(pack_k_onepass_batched_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)one_smem);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(KOP_CL, H, n_jobs);
    cfg.blockDim = dim3(KOP_WARPS * 32);
    cfg.dynamicSmemBytes = one_smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KOP_CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, pack_k_onepass_batched_kernel, jobs, kop_rows_per_cta(max_t_k), quads);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
    return launch_status();
  }
  if (D == 128) pack_k_minmax128_batched_kernel<<<dim3(pack_k_slabs(max_t_k), H, n_jobs), 128, 0, st>>>(jobs);
  else pack_k_minmax_batched_kernel<<<dim3(pack_k_slabs(max_t_k), H, n_jobs), 128, 0, st>>>(jobs);
  rc = launch_status();
  if (rc != RDKV_OK) return rc;
  pack_k_params_batched_kernel<<<dim3(H, n_jobs), 128, 0, st>>>(jobs);
  rc = launch_status();
  if (rc != RDKV_OK) return rc;
  const size_t smem = pack_k_quant_smem(max_d_pad, D == 128);
  if (cudaFuncSetAttribute(pack_k_quant_batched_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return launch_status();
  pack_k_quant_batched_kernel<<<dim3(pack_k_quant_ctas(max_t_k), H, n_jobs), PACKK_WARPS * 32, smem, st>>>(jobs);
  return launch_status();
}
