// Packed layer -> fp16 (K, V) on the stripe token axis: the inverse of the prefill packer, for
// fallback attention through an unpacked cache and for debugging.
//
// Reference behaviour (obkv_accel/packing.py:581-709 unpack_k_mixed, :1427-1444 unpack_v_segment;
// obkv_accel/trizone_decompress.py:43-183): value = half((float(code) - float(zp)) * float(scale)),
// K scattered back to the original channel of each kept slot (evicted channels are zeros), V rows
// in head-local segment order [2-bit | 4-bit | 8-bit], zero rows up to max_T_v, then the fp16
// Zone-B rows.  The subtraction is exact (small integers), so one fp32 multiply and one rounding
// to fp16 reproduce the reference bit for bit.
#include "rdkv_common.cuh"

namespace rdkv {

constexpr int UNPACK_WARPS = 8;
constexpr int UNPACK_MAX_D = 512;

__device__ __forceinline__ uint16_t dequant_h(unsigned code, uint16_t zp_bits, uint16_t sc_bits) {
  const float d = __fsub_rn((float)code, h2f(zp_bits));
  return __half_as_ushort(__float2half_rn(__fmul_rn(d, h2f(sc_bits))));
}

// grid (ceil(rows_out / UNPACK_WARPS), H_kv); one warp per stripe row.
__global__ void __launch_bounds__(UNPACK_WARPS * 32)
unpack_layer_kernel(rdkv_layer_view v, int D, const int64_t* __restrict__ k_sort_idx, int64_t k_sort_idx_head_stride,
                    const int32_t* __restrict__ k_ch_counts, int n_ch2, int n_ch4, int n_ch8,
                    uint16_t* __restrict__ k_out, uint16_t* __restrict__ v_out, int64_t out_head_stride, int rows_out) {
  __shared__ int16_t s_slot[UNPACK_MAX_D];                     // original channel -> slot in the padded order, -1: evicted
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n2p = v.n_ch2_pad, n4p = v.n_ch4_pad, n8p = v.n_ch8, d_pad = n2p + n4p + n8p;
  const int sub2 = n2p / 4, sub4 = n4p / 2;
  if (k_out != nullptr) {
    for (int c = threadIdx.x; c < D; c += blockDim.x) s_slot[c] = -1;
    __syncthreads();
    int c2 = n_ch2, c4 = n_ch4, c8 = n_ch8;
    if (k_ch_counts != nullptr) { c2 = k_ch_counts[h * 3 + 0]; c4 = k_ch_counts[h * 3 + 1]; c8 = k_ch_counts[h * 3 + 2]; }
    const int64_t* si = k_sort_idx + h * k_sort_idx_head_stride;
    for (int j = threadIdx.x; j < c2 + c4 + c8; j += blockDim.x) {
      const int slot = j < c2 ? j : j < c2 + c4 ? n2p + (j - c2) : n2p + n4p + (j - c2 - c4);
      const int64_t ch = si[j];
      if (ch >= 0 && ch < D) s_slot[ch] = (int16_t)slot;
    }
    __syncthreads();
  }
  const int row = blockIdx.x * UNPACK_WARPS + warp;
  if (row >= rows_out) return;

  if (k_out != nullptr) {
    uint16_t* dst = k_out + h * out_head_stride + (int64_t)row * D;
    const bool in_stripe = row < v.t_k && d_pad > 0;
    const uint8_t* r2 = v.k2 != nullptr ? v.k2 + h * v.k2_head_stride + (int64_t)row * sub2 : nullptr;
    const uint8_t* r4 = v.k4 != nullptr ? v.k4 + h * v.k4_head_stride + (int64_t)row * sub4 : nullptr;
    const uint8_t* r8 = v.k8 != nullptr ? v.k8 + h * v.k8_head_stride + (int64_t)row * n8p : nullptr;
    const uint16_t* sc = v.k_scale + (int64_t)h * d_pad;
    const uint16_t* zp = v.k_zp + (int64_t)h * d_pad;
    for (int c = lane; c < D; c += 32) {
      const int p = in_stripe ? s_slot[c] : -1;
      uint16_t out = 0;
      if (p >= 0) {
        unsigned code;
        if (p < n2p) code = (r2[p % sub2] >> (2 * (p / sub2))) & 3u;
        else if (p < n2p + n4p) { const int q = p - n2p; code = (r4[q % sub4] >> (4 * (q / sub4))) & 15u; }
        else code = r8[p - n2p - n4p];
        out = dequant_h(code, zp[p], sc[p]);
      }
      dst[c] = out;
    }
  }

  if (v_out != nullptr) {
    uint16_t* dst = v_out + h * out_head_stride + (int64_t)row * D;
    int n2 = v.n2, n4 = v.n4, n8 = v.n8;
    if (v.v_seg_bounds != nullptr) { n2 = v.v_seg_bounds[h * 3 + 0]; n4 = v.v_seg_bounds[h * 3 + 1]; n8 = v.v_seg_bounds[h * 3 + 2]; }
    const int t_v = n2 + n4 + n8;
    const int n16 = v.v16 == nullptr ? 0 : (v.n_v16 != nullptr ? v.n_v16[h] : v.n_v16_shared);
    if (row < t_v) {
      const int seg = row < n2 ? 0 : row < n2 + n4 ? 1 : 2;
      const int j = seg == 0 ? row : seg == 1 ? row - n2 : row - n2 - n4;
      const int sub = seg == 0 ? D / 4 : seg == 1 ? D / 2 : D;
      const uint8_t* src = seg == 0 ? v.v2 + h * v.v2_head_stride : seg == 1 ? v.v4 + h * v.v4_head_stride
                                                                             : v.v8 + h * v.v8_head_stride;
      src += (int64_t)j * sub;
      const uint16_t s = v.v_scale[h * v.v_meta_head_stride + row], z = v.v_zp[h * v.v_meta_head_stride + row];
      const int bits = seg == 0 ? 2 : seg == 1 ? 4 : 8;
      const unsigned mask = (1u << bits) - 1u;
      for (int c = lane; c < D; c += 32) {
        const unsigned code = (src[c % sub] >> (bits * (c / sub))) & mask;
        dst[c] = dequant_h(code, z, s);
      }
    } else if (row >= v.max_t_v && row < v.max_t_v + n16) {
      const uint16_t* src = v.v16 + h * v.v16_head_stride + (int64_t)(row - v.max_t_v) * D;
      for (int c = lane; c < D; c += 32) dst[c] = src[c];
    } else {
      for (int c = lane; c < D; c += 32) dst[c] = 0;
    }
  }
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int rdkv_unpack_layer(const rdkv_layer_view* view, int H_kv, int D, const int64_t* k_sort_idx,
                                 int64_t k_sort_idx_head_stride, const int32_t* k_ch_counts, int n_ch2, int n_ch4,
                                 int n_ch8, uint16_t* k_out, uint16_t* v_out, int64_t out_head_stride, int rows_out,
                                 void* stream) {
  if (view == nullptr || H_kv <= 0 || D <= 0 || rows_out < 0 || (k_out == nullptr && v_out == nullptr))
    return RDKV_ERR_BAD_ARG;
  if (D > UNPACK_MAX_D || (D & 3)) return RDKV_ERR_BAD_SHAPE;
  if (k_out != nullptr) {
    const int d_pad = view->n_ch2_pad + view->n_ch4_pad + view->n_ch8;
    if (d_pad > 0 && (view->k_scale == nullptr || view->k_zp == nullptr || k_sort_idx == nullptr)) return RDKV_ERR_BAD_ARG;
    if ((view->n_ch2_pad > 0 && view->k2 == nullptr) || (view->n_ch4_pad > 0 && view->k4 == nullptr) ||
        (view->n_ch8 > 0 && view->k8 == nullptr))
      return RDKV_ERR_BAD_ARG;
    if (n_ch2 < 0 || n_ch4 < 0 || n_ch8 < 0 || n_ch2 > view->n_ch2_pad || n_ch4 > view->n_ch4_pad || n_ch8 > view->n_ch8)
      return RDKV_ERR_BAD_ARG;
  }
  if (rows_out == 0) return RDKV_OK;
  if (H_kv > 65535) return RDKV_ERR_TOO_LARGE;
  dim3 grid((rows_out + UNPACK_WARPS - 1) / UNPACK_WARPS, H_kv);
  unpack_layer_kernel<<<grid, UNPACK_WARPS * 32, 0, (cudaStream_t)stream>>>(
      *view, D, k_sort_idx, k_sort_idx_head_stride, k_ch_counts, n_ch2, n_ch4, n_ch8, k_out, v_out, out_head_stride,
      rows_out);
  return launch_status();
}
