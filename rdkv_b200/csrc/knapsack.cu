// Batched Lagrangian bit allocator: one CTA per knapsack row, the row resident
// in shared memory, the whole multiplier search inside the kernel.
//
// Control flow and rounding follow the reference solver
// (knapsack_solver.py:121-248): cost = score*eps[n] + lambda*bits[n] with each
// product and the sum rounded to fp32 separately, first-index argmin, mean =
// exact integer sum / N in fp32, and the batch-wide exits of the lambda_hi
// doubling loop.
#include "rdkv_common.cuh"

namespace rdkv {

constexpr int KNAP_THREADS = 1024;
constexpr int KNAP_MAX_OPT = 8;
constexpr int KNAP_SMEM_ROW_BYTES = 200 * 1024;

struct KnapOpts {
  float bits[KNAP_MAX_OPT];
  float eps[KNAP_MAX_OPT];
  int ibits[KNAP_MAX_OPT];
  int n;
};

__device__ __forceinline__ int choose(float s, const float* se_unused, const KnapOpts& o, const float* lb) {
  int best = 0;
  float bc = __fadd_rn(__fmul_rn(s, o.eps[0]), lb[0]);
#pragma unroll
  for (int n = 1; n < KNAP_MAX_OPT; ++n) {
    if (n < o.n) {
      const float c = __fadd_rn(__fmul_rn(s, o.eps[n]), lb[n]);
      if (c < bc) { bc = c; best = n; }
    }
  }
  return best;
}

// Block-wide exact sum of the chosen bit costs for multiplier lam.
__device__ unsigned long long sweep_sum(const float* row, int len, float lam, const KnapOpts& o,
                                        unsigned long long* s_red) {
  float lb[KNAP_MAX_OPT];
#pragma unroll
  for (int n = 0; n < KNAP_MAX_OPT; ++n) lb[n] = n < o.n ? __fmul_rn(lam, o.bits[n]) : 0.f;
  unsigned int local = 0;
  for (int i = threadIdx.x; i < len; i += KNAP_THREADS) local += (unsigned)o.ibits[choose(row[i], nullptr, o, lb)];
  unsigned long long v = local;
#pragma unroll
  for (int ofs = 16; ofs > 0; ofs >>= 1) v += __shfl_xor_sync(0xffffffffu, v, ofs);
  __syncthreads();                       // s_red may still be read from the previous sweep
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long tot = 0;
  for (int w = 0; w < KNAP_THREADS / 32; ++w) tot += s_red[w];
  return tot;
}

__device__ __forceinline__ float mean_of(unsigned long long sum, int len) {
  return __fdiv_rn((float)sum, (float)len);
}

__device__ const float* stage_row(const float* grow, int len, float* smem_row, bool use_smem) {
  if (!use_smem) return grow;
  for (int i = threadIdx.x; i < len; i += KNAP_THREADS) smem_row[i] = grow[i];
  __syncthreads();
  return smem_row;
}

// Phase 1: lambda_hi seed and the number of doublings this row asks for (<= 40).
__global__ void __launch_bounds__(KNAP_THREADS)
knapsack_seed_kernel(const float* __restrict__ scores, int64_t row_stride, int len,
                     const float* __restrict__ budget, KnapOpts o, int use_smem,
                     float* __restrict__ lam0_out, int* __restrict__ ndbl_out) {
  extern __shared__ float smem_row[];
  __shared__ unsigned long long s_red[KNAP_THREADS / 32];
  __shared__ float s_max[KNAP_THREADS / 32];
  const int b = blockIdx.x;
  const float* row = stage_row(scores + (int64_t)b * row_stride, len, smem_row, use_smem != 0);
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < len; i += KNAP_THREADS) mx = fmaxf(mx, row[i]);
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = -INFINITY;
  for (int w = 0; w < KNAP_THREADS / 32; ++w) mx = fmaxf(mx, s_max[w]);
  const float lam0 = fmaxf(__fmul_rn(mx, 0.375f), 1e-8f);
  const float bud = budget[b];
  float lam = lam0;
  int k = 0;
  for (; k < 40; ++k) {
    const float avg = mean_of(sweep_sum(row, len, lam, o, s_red), len);
    if (!(avg > bud)) break;
    lam = __fmul_rn(lam, 2.0f);
  }
  if (threadIdx.x == 0) { lam0_out[b] = lam0; ndbl_out[b] = k; }
}

// Phase 2: batch-wide doubling count, lambda = 0 shortcut, bisection, final choice.
__global__ void __launch_bounds__(KNAP_THREADS)
knapsack_solve_kernel(const float* __restrict__ scores, int64_t row_stride, int n_rows, int len,
                      const float* __restrict__ budget, KnapOpts o, int max_iters, float tol,
                      int use_smem, const float* __restrict__ lam0_all,
                      const int* __restrict__ ndbl_all, int64_t* __restrict__ out) {
  extern __shared__ float smem_row[];
  __shared__ unsigned long long s_red[KNAP_THREADS / 32];
  const int b = blockIdx.x;
  // The reference doubles lambda_hi for all rows inside ONE loop that ends when no
  // row needs more or every lambda_hi reached 1e12; replay that loop on the seeds.
  int rounds = 40;
  for (int it = 0; it < 40; ++it) {
    int any_need = 0, all_big = 1;
    for (int r = threadIdx.x; r < n_rows; r += KNAP_THREADS) {
      const int k = ndbl_all[r];
      if (k > it) any_need = 1;
      const float lam = ldexpf(lam0_all[r], min(it + 1, k));
      if (!(lam >= 1e12f)) all_big = 0;
    }
    any_need = __syncthreads_or(any_need);
    all_big = __syncthreads_and(all_big);
    if (!any_need) { rounds = it; break; }
    if (all_big) { rounds = it + 1; break; }
  }
  const float* row = stage_row(scores + (int64_t)b * row_stride, len, smem_row, use_smem != 0);
  const float bud = budget[b];
  float lam_lo = 0.f;
  float lam_hi = ldexpf(lam0_all[b], min(rounds, ndbl_all[b]));
  float lam_final = 0.f;
  bool converged = !(mean_of(sweep_sum(row, len, 0.f, o, s_red), len) > bud);
  if (!converged) {
    float lam_mid = 0.f;
    for (int it = 0; it < max_iters; ++it) {
      lam_mid = __fdiv_rn(__fadd_rn(lam_lo, lam_hi), 2.0f);
      const float avg = mean_of(sweep_sum(row, len, lam_mid, o, s_red), len);
      const float rel = __fdiv_rn(fabsf(__fsub_rn(avg, bud)), fmaxf(bud, 1e-8f));
      if (rel < tol) { converged = true; break; }
      if (avg > bud) lam_lo = lam_mid; else lam_hi = lam_mid;
    }
    lam_final = lam_mid;                  // frozen value, or the last round's when never converged
  }
  float lb[KNAP_MAX_OPT];
#pragma unroll
  for (int n = 0; n < KNAP_MAX_OPT; ++n) lb[n] = n < o.n ? __fmul_rn(lam_final, o.bits[n]) : 0.f;
  int64_t* orow = out + (int64_t)b * len;
  for (int i = threadIdx.x; i < len; i += KNAP_THREADS) orow[i] = (int64_t)o.ibits[choose(row[i], nullptr, o, lb)];
}

// The single-row form of the reference (knapsack_solver.py:39-118) differs from the batched one in
// its arithmetic: the multiplier is bisected in double precision (Python floats) and enters the cost
// as its fp32 rounding, means and the tolerance test are compared in double, lambda_hi has no 1e-8
// floor and is doubled row by row until the mean fits or it reaches 1e12.  One CTA per row, rows
// independent.  (The reference does not terminate on a row whose scores are all zero while its
// cheapest option is above the budget — lambda_hi stays 0; the doubling here stops after 200 rounds.)
__global__ void __launch_bounds__(KNAP_THREADS)
knapsack_scalar_kernel(const float* __restrict__ scores, int64_t row_stride, int len,
                       const double* __restrict__ budget, KnapOpts o, int max_iters, double tol,
                       int use_smem, int64_t* __restrict__ out) {
  extern __shared__ float smem_row[];
  __shared__ unsigned long long s_red[KNAP_THREADS / 32];
  __shared__ float s_max[KNAP_THREADS / 32];
  const int b = blockIdx.x;
  const float* row = stage_row(scores + (int64_t)b * row_stride, len, smem_row, use_smem != 0);
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < len; i += KNAP_THREADS) mx = fmaxf(mx, row[i]);
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = -INFINITY;
  for (int w = 0; w < KNAP_THREADS / 32; ++w) mx = fmaxf(mx, s_max[w]);
  const double bud = budget[b];
  auto avg_at = [&](double lam) { return (double)mean_of(sweep_sum(row, len, (float)lam, o, s_red), len); };
  double lam_lo = 0.0, lam_hi = (double)mx * 0.375;
  for (int k = 0; k < 200 && avg_at(lam_hi) > bud && lam_hi < 1e12; ++k) lam_hi *= 2.0;
  double lam_final = 0.0;
  if (!(avg_at(0.0) <= bud)) {
    double lam_mid = 0.0;
    for (int it = 0; it < max_iters; ++it) {
      lam_mid = (lam_lo + lam_hi) / 2.0;
      const double avg = avg_at(lam_mid);
      if (fabs(avg - bud) / fmax(bud, 1e-8) < tol) break;
      if (avg > bud) lam_lo = lam_mid; else lam_hi = lam_mid;
    }
    lam_final = lam_mid;
  }
  float lb[KNAP_MAX_OPT];
#pragma unroll
  for (int n = 0; n < KNAP_MAX_OPT; ++n) lb[n] = n < o.n ? __fmul_rn((float)lam_final, o.bits[n]) : 0.f;
  int64_t* orow = out + (int64_t)b * len;
  for (int i = threadIdx.x; i < len; i += KNAP_THREADS) orow[i] = (int64_t)o.ibits[choose(row[i], nullptr, o, lb)];
}

}  // namespace rdkv

using namespace rdkv;

static int fill_options(KnapOpts& o, const float* option_bits, const float* option_eps, int n_options, int len) {
  o.n = n_options;
  float max_bit = 0.f;
  for (int n = 0; n < KNAP_MAX_OPT; ++n) {
    o.bits[n] = n < n_options ? option_bits[n] : 0.f;
    o.eps[n] = n < n_options ? option_eps[n] : 0.f;
    o.ibits[n] = (int)o.bits[n];
    if (n < n_options) {
      if (o.bits[n] < 0.f || (float)o.ibits[n] != o.bits[n]) return RDKV_ERR_BAD_ARG;
      max_bit = o.bits[n] > max_bit ? o.bits[n] : max_bit;
    }
  }
  if ((double)len * (double)max_bit >= 16777216.0) return RDKV_ERR_TOO_LARGE;
  return RDKV_OK;
}

extern "C" int rdkv_knapsack_rows(const float* scores, int64_t row_stride, int n_rows, int len, const double* budget,
                                  const float* option_bits, const float* option_eps, int n_options, int max_iters,
                                  double tol, int64_t* out, void* stream) {
  if (scores == nullptr || budget == nullptr || option_bits == nullptr || option_eps == nullptr || out == nullptr)
    return RDKV_ERR_BAD_ARG;
  if (n_rows < 0 || len <= 0 || max_iters < 0) return RDKV_ERR_BAD_ARG;
  if (n_options <= 0 || n_options > KNAP_MAX_OPT) return RDKV_ERR_BAD_SHAPE;
  if (n_rows == 0) return RDKV_OK;
  KnapOpts o;
  const int rc = fill_options(o, option_bits, option_eps, n_options, len);
  if (rc != RDKV_OK) return rc;
  const size_t row_bytes = (size_t)len * sizeof(float);
  const int use_smem = row_bytes <= (size_t)KNAP_SMEM_ROW_BYTES ? 1 : 0;
  const size_t smem = use_smem ? row_bytes : 0;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(knapsack_scalar_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KNAP_SMEM_ROW_BYTES);
  knapsack_scalar_kernel<<<n_rows, KNAP_THREADS, smem, (cudaStream_t)stream>>>(scores, row_stride, len, budget, o,
                                                                              max_iters, tol, use_smem, out);
  return launch_status();
}

extern "C" int rdkv_knapsack_batched(const float* scores, int64_t row_stride, int n_rows, int len,
                                     const float* budget, const float* option_bits,
                                     const float* option_eps, int n_options, int max_iters, float tol,
                                     int64_t* out, void* scratch, void* stream) {
  if (scores == nullptr || budget == nullptr || option_bits == nullptr || option_eps == nullptr ||
      out == nullptr || scratch == nullptr)
    return RDKV_ERR_BAD_ARG;
  if (n_rows < 0 || len <= 0 || max_iters < 0) return RDKV_ERR_BAD_ARG;
  if (n_options <= 0 || n_options > KNAP_MAX_OPT) return RDKV_ERR_BAD_SHAPE;
  if (n_rows == 0) return RDKV_OK;
  KnapOpts o;
  const int orc = fill_options(o, option_bits, option_eps, n_options, len);
  if (orc != RDKV_OK) return orc;
  const size_t row_bytes = (size_t)len * sizeof(float);
  const int use_smem = row_bytes <= (size_t)KNAP_SMEM_ROW_BYTES ? 1 : 0;
  const size_t smem = use_smem ? row_bytes : 0;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(knapsack_seed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KNAP_SMEM_ROW_BYTES);
    cudaFuncSetAttribute(knapsack_solve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KNAP_SMEM_ROW_BYTES);
  }
  float* lam0 = reinterpret_cast<float*>(scratch);
  int* ndbl = reinterpret_cast<int*>(lam0 + 2 * (size_t)n_rows);
  cudaStream_t st = (cudaStream_t)stream;
  knapsack_seed_kernel<<<n_rows, KNAP_THREADS, smem, st>>>(scores, row_stride, len, budget, o, use_smem, lam0, ndbl);
  int rc = launch_status();
  if (rc != RDKV_OK) return rc;
  knapsack_solve_kernel<<<n_rows, KNAP_THREADS, smem, st>>>(scores, row_stride, n_rows, len, budget, o,
                                                           max_iters, tol, use_smem, lam0, ndbl, out);
  return launch_status();
}

// ── allocation-free variant ──────────────────────────────────────────────────
// Some callers cannot provide the per-row scratch of rdkv_knapsack_batched because
// they are not allowed to allocate device memory at the point of the call: a
// prefill step that runs inside an engine's fixed memory plan after warm-up, or a
// plugin interface that hands over input and output buffers only.
// For them the scratch lives in this library's own device image: a file-scope
// array that every GPU loading the library carries until the process exits.
// (One warm-up call per device, made before the memory plan is frozen and before any
// stream capture, looks the array's address up and lets the runtime load the module;
// rows longer than 48 KiB also opt the kernels into large shared memory on that call,
// so the warm-up should use a row as long as the longest that will follow.)
constexpr int KNAP_STATIC_MAX_ROWS = 4096;                 // 3 words per row -> 48 KiB per GPU
static __device__ __align__(256) unsigned int g_knap_static_scratch[3 * KNAP_STATIC_MAX_ROWS];

#include <mutex>
namespace {
constexpr int KNAP_MAX_DEVICES = 64;
std::mutex g_knap_static_mutex;
void* g_knap_static_addr[KNAP_MAX_DEVICES] = {nullptr};   // device address of the array, per device
}  // namespace

extern "C" int rdkv_knapsack_static_max_rows(void) { return KNAP_STATIC_MAX_ROWS; }

extern "C" int rdkv_knapsack_batched_static(const float* scores, int64_t row_stride, int n_rows, int len,
                                            const float* budget, const float* option_bits,
                                            const float* option_eps, int n_options, int max_iters, float tol,
                                            int64_t* out, void* stream) {
  if (n_rows > KNAP_STATIC_MAX_ROWS) return RDKV_ERR_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= KNAP_MAX_DEVICES) {
    g_last_cuda_error = (int)e;
    return RDKV_ERR_NO_DEVICE;
  }
  void* scratch = nullptr;
  {
    // The array's name is only a host-side handle; the address a kernel can use is
    // looked up once per device, with that device current.
    std::lock_guard<std::mutex> lock(g_knap_static_mutex);
    if (g_knap_static_addr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_knap_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        g_last_cuda_error = (int)e;
        return RDKV_ERR_LAUNCH;
      }
      g_knap_static_addr[dev] = p;
    }
    scratch = g_knap_static_addr[dev];
  }
  return rdkv_knapsack_batched(scores, row_stride, n_rows, len, budget, option_bits, option_eps, n_options,
                               max_iters, tol, out, scratch, stream);
}
