// Fused split-sequence decode attention over the packed cache (sm_100a).
//
// One CTA = (view, KV head, chunk of live rows), 160 threads.  Warp 4 (the staging warp) works out
// the CTA's geometry, plans its tiles (up to 256 rows: six contiguous byte ranges each) and streams
// them into a 2-slot shared-memory ring with one bulk copy per range — the 8-bit and fp16 V rows as
// one tiled TMA box through a tensor map of the view's V tensor, 16 bytes wider than a row, so that
// the rows land at a pitch at which the P.V operand loads have no bank conflicts — completion
// counted on an mbarrier.  Warps 0-3 (the compute warps) fold the queries meanwhile and then work through the
// tiles, 32 rows (two 16-row MMA groups) per warp and step:
//   * q.K scores on the tensor cores (mma.sync m16n8k16, rows on M, query heads on N): packed
//     2/4/8-bit K codes are masked in place into fp16 SUBNORMAL integers (code * 2^-24, exact), so
//     unpacking is one AND per pair of codes; bit-position factors (4^v, 16) are folded into q*scale;
//   * an online softmax per query head in base 2 with a lazily moved reference maximum;
//   * exp2(s-m)*v_scale, transposed in registers (movmatrix), as the B operand of the P.V product
//     with V codes, again masked in place, as the A operand (channels on M, rows on K).
// Probabilities never leave registers.  Zero points are handled outside the products:
// sum_c zp*q*scale once per CTA (K side, reference "bias trick",
// obkv_accel/triton_k_kernel.py:14-16) and sum_t p*scale*zp per head (V side).
#include <cuda.h>   // CUtensorMap (the V tiles arrive through tensor maps; the encoder is looked up through the runtime)

#include <algorithm>
#include <cstring>
#include <type_traits>

#include "rdkv_common.cuh"

namespace rdkv {

#ifndef RDKV_FW
#define RDKV_FW 4
#endif
#ifndef RDKV_MINB
#define RDKV_MINB 3
#endif
#ifndef RDKV_FSTAGES
#define RDKV_FSTAGES 2
#endif
#ifndef RDKV_TILE_ROWS
#define RDKV_TILE_ROWS 256
#endif
constexpr int FW = RDKV_FW;            // consumer (compute) warps per CTA; one more warp stages the tiles
constexpr int CTA_THREADS = (FW + 1) * 32;
constexpr int FSTAGES = RDKV_FSTAGES;  // ring depth
constexpr int TILE_MAX = RDKV_TILE_ROWS;           // rows per tile (2-bit and 4-bit phases)
constexpr int V_PAD = 16;                          // bytes between V rows in a stage: rows 2j of a group fall on distinct banks
#ifndef RDKV_V_STAGE_PER_ROW
#define RDKV_V_STAGE_PER_ROW 72
#endif
constexpr int V_STAGE = RDKV_V_STAGE_PER_ROW * TILE_MAX;   // V payload bytes per stage (the 8-bit phase: TILE_MAX / 2 rows of 128 + 16 bytes)
constexpr int GH = 8;                  // query heads per CTA pass (N of the P.V product)
#ifndef RDKV_KB_MAX
#define RDKV_KB_MAX 24
#endif
#ifndef RDKV_DPAD_MAX
#define RDKV_DPAD_MAX 384
#endif
constexpr int KB_MAX = RDKV_KB_MAX;    // 16-channel blocks of the score product (3 segments x 128 channels at most)
constexpr int DPAD_MAX = RDKV_DPAD_MAX;  // padded channel slots of a view (n_ch2_pad + n_ch4_pad + n_ch8)
// dynamic shared memory behind the ring: folded queries in MMA fragment order, then the scratch the
// fold reads (the group's query rows as fp32, the head's K scales, zero points and channel permutation)
constexpr int QS_BYTES = KB_MAX * 32 * 8;
constexpr int FOLD_Q_BYTES = GH * 128 * 4;
constexpr int FOLD_META_BYTES = 3 * DPAD_MAX * 2;
constexpr int TAIL_BYTES = QS_BYTES + FOLD_Q_BYTES + FOLD_META_BYTES;
constexpr float TWO24 = 16777216.f;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr unsigned WAIT_LIMIT = 1u << 22;  // try_wait rounds before a compute warp gives up on a tile
constexpr float RESCALE_TH = 8.f;      // log2 slack before the running maximum is moved
constexpr float M_NONE = -1.0e30f;     // reference maximum of a head that has seen no live score yet (finite: no inf - inf)

// (phase 4 = the uncompressed tail: plain K and V rows of 256 bytes each share the V area of a stage)
__host__ __device__ constexpr int phase_tile_rows(int p) {
  return p < 2 ? TILE_MAX : p == 2 ? TILE_MAX / 2 : p == 3 ? TILE_MAX / 4 : TILE_MAX / 8;
}
__host__ __device__ constexpr int phase_row_bytes(int p) { return p == 0 ? 32 : p == 1 ? 64 : p == 2 ? 128 : 256; }
// Distance of consecutive V rows in a stage.  A thread of the P.V product reads the same bytes of
// rows 2j (j = its place in its quad): with rows of 32 .. 256 bytes laid end to end the four rows
// of a quad would share their banks; 16 bytes more per row puts them 32 bytes apart modulo 128.
// (The tail's plain rows keep their 256 bytes.)
#ifndef RDKV_STATIC_ROUNDS
#define RDKV_STATIC_ROUNDS 1
#endif
#ifndef RDKV_V_PAD_FROM
#define RDKV_V_PAD_FROM 2
#endif
// First V phase whose rows are spaced: the 8-bit rows (128 bytes) and the fp16 rows (256 bytes), whose
// loads are 32 per 32-row block and conflict four ways when the rows lie end to end.  The 2-bit and
// 4-bit rows (8 and 16 loads per block) stay dense: as 48- and 80-byte box rows they travel more
// slowly than in one bulk copy (measured: spacing all four phases is slower than spacing none).
constexpr int V_PAD_FROM = RDKV_V_PAD_FROM;
__host__ __device__ constexpr int phase_pitch(int p) {
  return (p == 4 || p < V_PAD_FROM) ? phase_row_bytes(p) : phase_row_bytes(p) + V_PAD;
}
static_assert(phase_tile_rows(0) * phase_pitch(0) <= V_STAGE && phase_tile_rows(1) * phase_pitch(1) <= V_STAGE &&
              phase_tile_rows(2) * phase_pitch(2) <= V_STAGE && phase_tile_rows(3) * phase_pitch(3) <= V_STAGE,
              "a tile's V rows fit the V area at their padded pitch");

__host__ __device__ inline int align16i(int x) { return (x + 15) & ~15; }
__host__ __device__ inline int align128i(int x) { return (x + 127) & ~127; }

struct StageLayout {                   // byte offsets inside one stage
  int v, k2, k4, k8, sc, zp, total;
};

__host__ __device__ inline StageLayout stage_layout(int sub2, int sub4, int n8) {
  StageLayout L;
  L.v = 0;
  L.k2 = V_STAGE + 32;
  L.k4 = L.k2 + align16i(TILE_MAX * sub2) + 48;
  L.k8 = L.k4 + align16i(TILE_MAX * sub4) + 48;
  L.sc = L.k8 + align16i(TILE_MAX * n8) + 48;
  L.zp = L.sc + TILE_MAX * 2 + 32;
  L.total = L.zp + TILE_MAX * 2 + 32;
  return L;
}

__host__ __device__ inline int stage_capacity(int k_row_bytes_max) {
  return V_STAGE + 32 + TILE_MAX * k_row_bytes_max + 3 * 64 + 2 * (TILE_MAX * 2 + 32);
}

// ── PTX wrappers ─────────────────────────────────────────────────────────────
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte global -> shared copy (L2 only); src and dst are 16-byte aligned.
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Same, reading only the first src_bytes (< 16) bytes and zero-filling the rest.
__device__ __forceinline__ void cp16_partial(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// mbarrier (shared memory, CTA scope).  A tile's arrival is signalled asynchronously: every
// staging lane posts one arrival that fires when its cp.async copies have landed.
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Adds `bytes` to the transaction count the current phase waits for (no arrival).
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16) whose
// completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Same with an L2 eviction policy for the lines it reads.
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
               : "memory");
}
// One box of a 2-D tensor map (x in elements of the map's type, y = row) into shared memory (128-byte
// aligned), counted in bytes on `bar` like a bulk copy; rows and columns past the tensor arrive as zeros.
__device__ __forceinline__ void tma_g2s_2d(uint32_t dst, const void* map, int x, int y, uint64_t* bar, uint64_t pol) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(pol)
               : "memory");
}
// The two copies as predicated instructions: a warp whose lanes issue different kinds of copy (or
// none) stays on one straight path.
__device__ __forceinline__ void bulk_g2s_hint_if(bool on, uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %5, 0;\n"
      " @p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n}\n"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol), "r"((uint32_t)on)
      : "memory");
}
__device__ __forceinline__ void tma_g2s_2d_if(bool on, uint32_t dst, const void* map, int x, int y, uint64_t* bar, uint64_t pol) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %6, 0;\n"
      " @p cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;\n}\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(pol), "r"((uint32_t)on)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_on_copies(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Named barriers: `count` threads must arrive (bar.arrive or bar.sync) to release the waiters.
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Same with a zero accumulator input: starts a chain without materialising zeros in registers.
__device__ __forceinline__ void mma16816_z(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  return __byte_perm(a, b, sel);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// Transpose of an 8x8 matrix of 16-bit elements held one row pair per thread (thread
// 4r+j: row r, columns 2j and 2j+1): afterwards thread 4r+j holds column r, rows 2j, 2j+1.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
// Loads of the small per-launch tables (view records, prepared tables) ask L2 to keep their lines
// over the packed payload that streams through it (evict_last); the payload's bulk copies ask for
// evict_first.
#ifndef RDKV_L2HINT
#define RDKV_L2HINT 1
#endif
__device__ __forceinline__ uint64_t l2_policy_keep() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_stream() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ int ldg_keep(const int* a) {
#if RDKV_L2HINT
  int x;
  asm volatile("ld.global.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(x) : "l"(a), "l"(l2_policy_keep()));
  return x;
#else
  return *a;
#endif
}
__device__ __forceinline__ int4 ldg_keep4(const int4* a) {
#if RDKV_L2HINT
  int4 x;
  asm volatile("ld.global.L2::cache_hint.v4.b32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w)
               : "l"(a), "l"(l2_policy_keep()));
  return x;
#else
  return *a;
#endif
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  const __half2 c = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&c);
}
__device__ __forceinline__ float pow2i(int e) { return __int_as_float((127 + e) << 23); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Shared-memory loads through 32-bit shared-window addresses (IMM: constant byte offset).
template <int IMM = 0>
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(IMM));
  return v;
}
template <int IMM = 0>
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(a), "n"(IMM));
  return v;
}
template <int IMM = 0>
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(IMM));
  return v;
}
// 32 bits starting at an arbitrary byte address of shared memory (two aligned loads).
__device__ __forceinline__ uint32_t lds32_unaligned(uint32_t a) {
  const uint32_t lo = lds32(a & ~3u), hi = lds32<4>(a & ~3u);
  return __funnelshift_r(lo, hi, (a & 3u) * 8);
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// ── K channel-slot map: which padded channel slot feeds MMA k-index e of thread j ──
// e = 0..3 stands for k = 2j, 2j+1, 2j+8, 2j+9.  Returns the slot or -1, and the
// power-of-two factor the masked code carries (folded into q*scale).
struct KDims { int sub2, sub4, n8, n2p, n4p, nsp2, nsp4, nkb8, nkb; };

__host__ __device__ inline KDims k_dims(int n2p, int n4p, int n8) {
  KDims d;
  d.n2p = n2p; d.n4p = n4p; d.n8 = n8;
  d.sub2 = n2p >> 2; d.sub4 = n4p >> 1;
  d.nsp2 = (d.sub2 + 7) >> 3; d.nsp4 = (d.sub4 + 15) >> 4; d.nkb8 = (n8 + 15) >> 4;
  d.nkb = 2 * d.nsp2 + 2 * d.nsp4 + d.nkb8;
  return d;
}

__device__ inline int k_slot(const KDims& d, int kb, int j, int e, float* factor) {
  if (kb < 2 * d.nsp2) {
    const int s = kb >> 1, half = kb & 1;
    const int i = 8 * s + 2 * j + (e & 1), v = 2 * half + (e >> 1);
    *factor = (float)(1 << (2 * v));
    return i < d.sub2 ? i + v * d.sub2 : -1;
  }
  kb -= 2 * d.nsp2;
  if (kb < 2 * d.nsp4) {
    const int s = kb >> 1, half = kb & 1;
    const int i = 16 * s + 4 * j + half + 2 * (e & 1), hi = e >> 1;
    *factor = hi ? 16.f : 1.f;
    return i < d.sub4 ? d.n2p + i + hi * d.sub4 : -1;
  }
  kb -= 2 * d.nsp4;
  const int i = 16 * kb + 4 * j + (e >> 1) + 2 * (e & 1);
  *factor = 1.f;
  return i < d.n8 ? d.n2p + d.n4p + i : -1;
}

// Per (view, KV head) record of a prepared table (rdkv_decode_prepare): the head's row counts and
// whether every byte range of the whole head lies on 16-byte blocks inside its tensor (then so
// does every sub-range a chunk may take), and per V phase where its rows start in every tensor, so
// that a chunk's geometry is a few integer operations on one record.  16-byte aligned.
struct __align__(16) PhaseRec {                 // one V phase (2-bit, 4-bit, 8-bit, fp16 rows) of the head
  int b_lo, b_hi, v_row, pad1;                   // its live-row range; row b_lo's number in the phase's tensor map (-1: no map)
  const unsigned char *k2, *k4, *k8, *vrow, *sc, *zp;   // addresses of row b_lo in the K streams, the V tensor, V scale / zero point
};
struct __align__(16) UnitRec {
  int n2, n4, n8, n16;
  int flags, nkb, n_ch2_pad, n_ch4_pad;
  int n_ch8, max_t_v;
  unsigned vmaps_lo, vmaps_hi;                   // the view's four tensor maps (128 bytes each, by phase), or 0
  PhaseRec ph[4];
};
static_assert(sizeof(PhaseRec) == 64 && sizeof(UnitRec) == 304, "prepared-table records are read as int4 words");
// One slot quadruple of the prepared K table: what thread `lane` of 16-channel block `kb` needs to
// fold its four query elements — original channels, zero points (integers 0..255) and fp16 scales
// (0 for a pad slot).  16 bytes; [unit][kb][lane].
struct __align__(16) KSlotRec { uint32_t perm4, zp4, sc01, sc23; };

// Sequence parts: a head's rows are shared out phase by phase (every part gets its share of the
// 2-bit, of the 4-bit, of the 8-bit and of the fp16 rows, so the parts read about the same bytes);
// part i of `parts` takes rows [part_cut(n, i), part_cut(n, i + 1)) of a phase of n rows.
__host__ __device__ inline int part_cut(int n, int i, int parts) {
  return i >= parts ? n : (int)(((int64_t)n * i / parts) & ~31);
}

// Accumulator unit exponent: true value = acc * 2^E(phase, v), v = m-tile & 3.
__device__ __forceinline__ int acc_exp(int phase, int v) {
  return phase == 0 ? 24 - 2 * v : phase == 1 ? 24 - 4 * (v >> 1) : phase == 2 ? 24 : 0;
}

// Everything a worker needs to find and stage its tiles; filled once per CTA.
struct CtaGeom {
  int lo[5], hi[5];                    // live-row range of this CTA per phase (2-bit, 4-bit, 8-bit, fp16, uncompressed tail)
  int first_tile[6];                   // [number of phases] = all tiles of the CTA, or -1: the view does not fit the launch
  int fast;                            // every staged range lies on whole 16-byte blocks of its tensor
  int64_t krow[4];                     // stripe row of live row lo[p]
  const unsigned char* k2[4];          // address of the K rows of live row lo[p]
  const unsigned char* k4[4];
  const unsigned char* k8[4];
  const unsigned char* vrow[5];        // address of the V row of live row lo[p]
  int vrow_idx[4];                     // its row number in the phase's tensor map, or -1
  const unsigned char* vmaps;          // the view's four tensor maps (by phase), or null
  const unsigned char* krow_tail;      // address of the plain K row of tail row lo[4]
  const unsigned char* sc[3];
  const unsigned char* zp[3];
};

struct TileDesc { int phase, row0, n; };   // row0: offset from lo[phase]

// What the staging warp tells the compute warps about the tile in a ring slot (16 bytes).
struct __align__(16) TileInfo {
  int phase, n;
  uint32_t offs;                       // six nibbles: byte offset (0..15) of row 0 inside the k2, k4, k8, v, scale, zp areas
  int krow0;                           // stripe row of row 0 (mask column)
};
// One byte range of a tile as the staging warp plans it (16 bytes), and a planned tile.
struct __align__(16) RangePlan { const unsigned char* src; int len; uint32_t dst_off; };
struct __align__(16) TilePlan { RangePlan rg[6]; TileInfo info; };
constexpr int PLAN_TILES = 32;         // tiles planned per round (one per staging lane)

template <int NPH>
__device__ __forceinline__ TileDesc tile_of(const CtaGeom& G, int idx) {
  TileDesc t;
  int p = 0;
#pragma unroll
  for (int k = 1; k < NPH; ++k)
    if (idx >= G.first_tile[k]) p = k;
  t.phase = p;
  const int tr = phase_tile_rows(p);
  t.row0 = (idx - G.first_tile[p]) * tr;
  t.n = min(tr, G.hi[p] - G.lo[p] - t.row0);
  return t;
}

// True when the 16-byte blocks covering [lo, hi) are all inside [t_lo, t_hi).
__device__ __forceinline__ bool blocks_inside(const unsigned char* lo, const unsigned char* hi,
                                              const unsigned char* t_lo, const unsigned char* t_hi) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(lo) & ~(uintptr_t)15;
  const uintptr_t b = (reinterpret_cast<uintptr_t>(hi) + 15) & ~(uintptr_t)15;
  return a >= reinterpret_cast<uintptr_t>(t_lo) && b <= reinterpret_cast<uintptr_t>(t_hi);
}

// Stage one byte range whose covering 16-byte blocks may stick out of its tensor [t_lo, t_hi) (a
// tensor start or end that is not 16-byte aligned) with per-lane 16-byte cp.async copies: the
// byte at global address x lands at dst + (x - (src & ~15)); a block crossing the end is read
// partially and zero-filled, a block crossing the start is copied byte by byte.
__device__ __noinline__ void stage_range_guarded(unsigned char* dst_ptr, const unsigned char* src, int len,
                                                 const unsigned char* t_lo, const unsigned char* t_hi, int tid,
                                                 int nt) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(src), a0 = a & ~(uintptr_t)15;
  const uintptr_t tl = reinterpret_cast<uintptr_t>(t_lo), th = reinterpret_cast<uintptr_t>(t_hi);
  const int nblk = (int)((((a + len + 15) & ~(uintptr_t)15) - a0) >> 4);
  const uint32_t dst = smem_u32(dst_ptr);
#pragma unroll 1
  for (int b = tid; b < nblk; b += nt) {
    const uintptr_t lo = a0 + 16 * (uintptr_t)b;
    if (lo < tl) {
      for (uintptr_t x = tl; x < lo + 16 && x < th; ++x) dst_ptr[x - a0] = *reinterpret_cast<const unsigned char*>(x);
    } else if (lo + 16 > th) {
      if (th > lo) cp16_partial(dst + 16 * b, reinterpret_cast<const void*>(lo), (int)(th - lo));
    } else {
      cp16(dst + 16 * b, reinterpret_cast<const void*>(lo));
    }
  }
}

// V rows of a tile into a stage at their padded pitch by the lanes of the staging warp (what a
// tensor map does in one instruction when the table has one): 16-byte copies when the rows are
// aligned, bytes otherwise.  The rows lie inside their tensor.
__device__ __noinline__ void stage_v_rows_padded(unsigned char* dst_ptr, const unsigned char* src, int n_rows, int row_bytes,
                                                 int pitch, int lane) {
  if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const int per = row_bytes >> 4;
    const uint32_t dst = smem_u32(dst_ptr);
#pragma unroll 1
    for (int b = lane; b < n_rows * per; b += 32) {
      const int row = b / per, c = b - row * per;
      cp16(dst + row * pitch + 16 * c, src + 16 * (int64_t)b);
    }
  } else {
#pragma unroll 1
    for (int x = lane; x < n_rows * row_bytes; x += 32) {
      const int row = x / row_bytes;
      dst_ptr[row * pitch + (x - row * row_bytes)] = src[x];
    }
  }
}

// Last step of a CTA: the partial results of the compute warps (o in `red` [FW][GH][128], and per
// warp and head m, l and the zero-point term in `ml` [FW][GH][3]) become the CTA's result.  Kept
// out of line so that its registers do not weigh on the main loop.  how: 0 = (m, l, o) record,
// 1 = normalised output, 2 = plain sum (weights were given).
// (COMPUTE_ONLY: called by the compute warps alone — their named barrier instead of __syncthreads.)
template <bool COMPUTE_ONLY>
__device__ __forceinline__ void epi_sync() {
  if (COMPUTE_ONLY) bar_sync(1 + FSTAGES, FW * 32); else __syncthreads();
}

template <bool COMPUTE_ONLY>
__device__ __noinline__ void final_merge(const float* red, const float* ml, int gcnt, int how, float* out_rows,
                                         float* rec0, int64_t rec_stride) {
  // Warp w of the first four takes heads w, w + 4; a lane four channels.  Every lane works out its
  // head's maximum, the weight of every compute warp's partial, l and the zero-point term for itself
  // (broadcast reads), so the merge needs no barrier of its own; kept small: it runs once per item,
  // from a cold instruction cache.
  const int t = threadIdx.x;
  if (t >= 128) return;
  const int d0 = (t & 31) * 4;
#pragma unroll 1
  for (int hq = t >> 5; hq < gcnt; hq += 4) {
    float M = M_NONE;
#pragma unroll
    for (int w = 0; w < FW; ++w) M = fmaxf(M, ml[(w * GH + hq) * 3]);
    float L = 0.f, Z = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < FW; ++w) {
      const float wgt = ex2(ml[(w * GH + hq) * 3] - M);
      L = fmaf(ml[(w * GH + hq) * 3 + 1], wgt, L);
      Z = fmaf(ml[(w * GH + hq) * 3 + 2], wgt, Z);
      const float4 x = *reinterpret_cast<const float4*>(red + (w * GH + hq) * D + d0);
      o.x = fmaf(x.x, wgt, o.x); o.y = fmaf(x.y, wgt, o.y); o.z = fmaf(x.z, wgt, o.z); o.w = fmaf(x.w, wgt, o.w);
    }
    o.x -= Z; o.y -= Z; o.z -= Z; o.w -= Z;
    if (how == 2) {
      *reinterpret_cast<float4*>(out_rows + hq * D + d0) = o;
    } else if (how == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      *reinterpret_cast<float4*>(out_rows + hq * D + d0) = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    } else {
      float* rec = rec0 + hq * rec_stride;
      *reinterpret_cast<float4*>(rec + 4 + d0) = o;
      if (d0 == 0)                                         // m in natural-log units; -inf marks an empty record
        *reinterpret_cast<float4*>(rec) = make_float4(M <= M_NONE ? -INFINITY : M * LN2, L, 0.f, 0.f);
    }
  }
}

// Chunked units without a second launch: every CTA of a unit (view, KV head, head group) calls
// this after it has written its chunk's records.  The CTAs count themselves on the unit's arrival
// counter; the one that finds it has arrived last merges the unit's n_chunks records per query
// head, in chunk order (so the result does not depend on who arrived last), into the normalised
// output or one un-normalised record, and puts the counter back to zero for the next launch.
// Nobody waits for anybody.  (Measured against a variant in which the CTA of the last chunk
// polls the counter and the others leave without reading it: no difference.)
// row0: index of the unit's first query head among all (view, head) rows.
template <bool COMPUTE_ONLY>
__device__ __noinline__ void chunk_merge(const float* partials, int* counter, int n_chunks, int gcnt,
                                         int64_t row0, float* out, float* merged) {
  __shared__ int s_last;
  const int tid = threadIdx.x;
  epi_sync<COMPUTE_ONLY>();                                         // the CTA's record stores are ordered before thread 0's fence
  if (tid == 0) {
    __threadfence();
    const int old = atomicAdd(counter, 1);
    s_last = old == n_chunks - 1;
    if (s_last) { *counter = 0; __threadfence(); }         // acquire side: the other CTAs' records
  }
  epi_sync<COMPUTE_ONLY>();
  if (!s_last) return;
  // thread = (query head slot, channel quarter): every load of the unit's records is in flight at once
  for (int base_hq = 0; base_hq < gcnt; base_hq += 4) {
    const int hq = base_hq + (tid >> 5);
    if (tid >= 128 || hq >= gcnt) continue;
    const int d0 = (tid & 31) * 4;
    const float* base = partials + (row0 + hq) * n_chunks * RDKV_PARTIAL_STRIDE;
    float M = -INFINITY, L = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
    for (int s0 = 0; s0 < n_chunks; s0 += 4) {             // four records in flight at a time, merged in chunk order
      float m[4], l[4];
      float4 x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool ok = s0 + i < n_chunks;
        const float* rec = base + (s0 + i) * RDKV_PARTIAL_STRIDE;
        m[i] = ok ? __ldcg(rec) : -INFINITY;
        l[i] = ok ? __ldcg(rec + 1) : 0.f;
        x[i] = ok ? __ldcg(reinterpret_cast<const float4*>(rec + 4 + d0)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (m[i] == -INFINITY) continue;
        const float Mn = fmaxf(M, m[i]);
        const float a = exp2f((M - Mn) * LOG2E), b = exp2f((m[i] - Mn) * LOG2E);
        L = L * a + l[i] * b;
        o.x = o.x * a + x[i].x * b; o.y = o.y * a + x[i].y * b; o.z = o.z * a + x[i].z * b; o.w = o.w * a + x[i].w * b;
        M = Mn;
      }
    }
    if (out != nullptr) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      *reinterpret_cast<float4*>(out + (row0 + hq) * D + d0) = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    } else {
      float* rec = merged + (row0 + hq) * RDKV_PARTIAL_STRIDE;
      *reinterpret_cast<float4*>(rec + 4 + d0) = o;
      if (d0 == 0) *reinterpret_cast<float4*>(rec) = make_float4(M, L, 0.f, 0.f);
    }
  }
}

// What a CTA's last step needs, parked in shared memory at its start so that it does not occupy
// registers across the tile loop.
struct EpiInfo {
  float* out_rows;                     // normalised output rows of this CTA's query heads
  float* rec0;                         // record of its first query head (records of the next heads rec_stride floats on)
  int64_t rec_stride;
  int64_t row0;                        // index of its first query head among all (view, head) rows
  int how, gcnt, n_chunks, unit_y;
};

// MODE_ATTN: the whole attention block.  MODE_SCORES: only the q.K scores of the live rows, written
// to aux[(query head) * aux_stride + stripe row] for stripe rows < t_eff (the K kernel of the
// two-stage interface; V is not read).  MODE_WEIGHTS: the softmax weights are given in
// aux[(query head) * aux_stride + stripe row]; only sum_t w.V is computed (the V kernel of the
// two-stage interface; K is not read), records carry m = 0 and l = 1 in chunk 0 so that the
// combine kernel adds the chunks up.
// MODE_ATTN_TAIL: MODE_ATTN over the packed zones plus, in the same softmax, the uncompressed tail
// of decode-appended tokens (a fifth tile phase of plain 16-bit K and V rows) and the token being
// decoded, with the rotary embedding of the query rows and of the new key row applied on the way
// in (TailArgs).  A separate instantiation: the other modes' code is not touched by it.
constexpr int MODE_ATTN = 0, MODE_SCORES = 1, MODE_WEIGHTS = 2, MODE_ATTN_TAIL = 3;
constexpr int TAIL_TILE = TILE_MAX / 8;             // tail rows per tile: K rows and V rows fill the V area together
constexpr int TAILQ_BYTES = 8 * 32 * 8;             // the queries as fp16 B fragments of the tail's score product
constexpr int TAIL_EXTRA_BYTES = TAILQ_BYTES + 2 * 128 * 4 + 64;   // + new key row, new value row (fp32), its scores
static_assert(2 * TAIL_TILE * 256 <= V_STAGE, "a tail tile's K and V rows share the V area");

using TailArgs = rdkv_tail_args;

template <int MODE>
#ifdef RDKV_MAXNREG
__global__ void __maxnreg__(RDKV_MAXNREG)
#else
__global__ void __launch_bounds__(CTA_THREADS, RDKV_MINB)
#endif
decode_fused_kernel(const rdkv_layer_view* __restrict__ views, const void* __restrict__ q, int q_dtype,
                    int H_q, int g, int chunk_rows, int k_chunks, int n_whole, int stage_bytes,
                    float* __restrict__ partials, float* __restrict__ out, int* __restrict__ status,
                    float* __restrict__ aux, int64_t aux_stride, int t_eff,
                    const UnitRec* __restrict__ unit_recs, const KSlotRec* __restrict__ kslots, int nkb_max,
                    int* __restrict__ unit_ctr, float* __restrict__ merged, int row_begin, int row_end,
                    int part, int parts, const TailArgs ta) {
  constexpr bool TAIL = MODE == MODE_ATTN_TAIL;
  constexpr bool ATTN = MODE == MODE_ATTN || TAIL;
  constexpr int NPH = TAIL ? 5 : 4;                // tile phases
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ rdkv_layer_view v;
  __shared__ CtaGeom G;
  __shared__ float s_ml[FW][GH][3];               // per warp: m, l, zero-point term
  __shared__ float s_bias[FW][GH];                // zero-point bias of the folded queries: the warps' partial sums
  __shared__ EpiInfo s_epi;
  __shared__ TileInfo s_tile[FSTAGES];
  __shared__ TilePlan s_plan[PLAN_TILES];          // private to the staging warp
  __shared__ __align__(8) uint64_t s_full[FSTAGES];   // tile in slot s has landed

  // Work items, one per CTA, in launch order: the first n_whole units (view, KV head, group of
  // query heads) whole, then every remaining unit as k_chunks chunks of chunk_rows live rows.
  // (Whole units first: the chunks fill the last, partly empty round of CTAs.)
  const int n_hgrp = (g + GH - 1) / GH;
  const int hy = (H_q / g) * n_hgrp;
  int unit_y, chunk, n_chunks;
  if ((int)blockIdx.x < n_whole) {
    unit_y = blockIdx.x; chunk = 0; n_chunks = 1;
  } else {
    const int jj = blockIdx.x - n_whole;
    unit_y = n_whole + jj / k_chunks; chunk = jj % k_chunks; n_chunks = k_chunks;
  }
  const int view_idx = unit_y / hy;
  const int h = (unit_y % hy) / n_hgrp, hgrp = (unit_y % hy) % n_hgrp;
  const int gh0 = hgrp * GH, gcnt = min(GH, g - gh0);     // query heads [gh0, gh0+gcnt) of this KV head
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, j = lane & 3;
  const int hq0 = h * g + gh0;                             // first query head handled here

  const uint32_t smem0 = smem_u32(smem_raw);
  const uint32_t qs_base = smem0 + FSTAGES * stage_bytes;  // uint2 qsA[nkb][32]
  unsigned char* tail = smem_raw + (size_t)FSTAGES * stage_bytes;
  // (a launch with a prepared table knows the largest number of K blocks of its views: the folded
  // queries take that many blocks of 256 bytes, not the 24 a view may have at most)
  const int qs_bytes = (nkb_max > 0 ? min(nkb_max, KB_MAX) : KB_MAX) * 256;
  const int tail_bytes = qs_bytes + FOLD_Q_BYTES + FOLD_META_BYTES;
  uint2* qsA = reinterpret_cast<uint2*>(tail);
  float* f_q = reinterpret_cast<float*>(tail + qs_bytes);                   // [gcnt][128] query rows as fp32
  uint16_t* f_sc = reinterpret_cast<uint16_t*>(tail + qs_bytes + FOLD_Q_BYTES);   // [d_pad] K scales (fp16 bits; launches without a prepared table)
  uint16_t* f_zp = f_sc + DPAD_MAX;                                         // [d_pad] K zero points (fp16 bits)
  uint16_t* f_pm = f_zp + DPAD_MAX;                                         // [d_pad] original channel of each slot

  // ── first round trip.  Compute warps: the view record, this thread's K slots of the prepared
  //    table and the group's query rows.  Staging warp: the unit's record of the prepared table,
  //    from which it works out the CTA's geometry without waiting for anything else.  Nothing
  //    here depends on anything but the launch arguments. ──
  // named barrier ids: FREE[s] = 1 + s (slot s may be refilled); COMPUTE: the compute warps among
  // themselves; GEOM: the staging warp has published the CTA's geometry; VIEW: the view record
  // and the query rows are in shared memory
  constexpr int BAR_FREE = 1, BAR_COMPUTE = 1 + FSTAGES, BAR_GEOM = 2 + FSTAGES, BAR_VIEW = 3 + FSTAGES;
  const bool prepared = unit_recs != nullptr;
  const int64_t unit = (int64_t)view_idx * (H_q / g) + h;
  KSlotRec km0 = {0u, 0u, 0u, 0u}, km1 = km0;              // this thread's slots of blocks warp, warp + FW
  int n2p = 0, n4p = 0, n8c = 0;                           // padded channel counts of the view
  bool geom_done = false;
  int n_tail = 0;                                          // live rows of the uncompressed tail of this view
  // the tail's share of this CTA, from the rows pn0..pn3 the part has of the four packed phases:
  // window [lo, hi) in the part's row numbering, first tail row d, tiles
  struct TailGeom { int lo, hi, d, tiles; };
  auto tail_geom = [&](int pn0, int pn1, int pn2, int pn3, int c0, int c1) {
    const int ps4 = part_cut(n_tail, part, parts), pn4 = part_cut(n_tail, part + 1, parts) - ps4;
    const int lb4 = pn0 + pn1 + pn2 + pn3;
    TailGeom t;
    t.lo = max(lb4, c0); t.hi = max(t.lo, min(lb4 + pn4, c1));
    t.d = ps4 + (t.lo - lb4);
    t.tiles = (t.hi - t.lo + TAIL_TILE - 1) / TAIL_TILE;
    return t;
  };
  auto tail_row = [&](const void* base, int row) {         // address of a row of this (view, KV head)'s tail buffer
    return reinterpret_cast<const unsigned char*>(base) +
           ((int64_t)view_idx * ta.view_stride + (int64_t)h * ta.head_stride + (int64_t)row * D) * 2;
  };
  if (TAIL)
    n_tail = ta.n_new_per_view != nullptr ? min(max(ldg_keep(ta.n_new_per_view + view_idx), 0), ta.cap) : ta.n_new;
  if (warp == FW) {
    if (lane < FSTAGES) mbar_init(&s_full[lane], 64);      // per staging lane: one plain + one copy-completion arrival
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    if (prepared) {
      const int4* up = reinterpret_cast<const int4*>(unit_recs + unit);
      const int p = lane & 3;
      const int4 h1 = ldg_keep4(up + 1), h2 = ldg_keep4(up + 2);
      const int4 a0 = ldg_keep4(up + 3 + 4 * p), a1 = ldg_keep4(up + 4 + 4 * p), a2 = ldg_keep4(up + 5 + 4 * p),
                 a3 = ldg_keep4(up + 6 + 4 * p);
      if (h1.x & 1) {                                      // every range of the head lies on whole 16-byte blocks
        bar_arrive(BAR_VIEW, CTA_THREADS);
        n2p = h1.z; n4p = h1.w; n8c = h2.x;
        const KDims kq = k_dims(n2p, n4p, n8c);
        const StageLayout SQ = stage_layout(kq.sub2, kq.sub4, kq.n8);
        const bool fits_q = SQ.total <= stage_bytes && kq.n2p + kq.n4p + kq.n8 > 0 &&
                            kq.n2p + kq.n4p + kq.n8 <= DPAD_MAX && kq.nkb <= KB_MAX;
        const int c0 = row_begin + chunk * chunk_rows, c1 = n_chunks == 1 ? row_end : min(c0 + chunk_rows, row_end);
        // this part's share of the phase, then the chunk's window of the part's rows (numbered phase
        // after phase): lo, hi in that numbering; d = first row's offset from the phase's first row
        const int np = a0.y - a0.x, ps = part_cut(np, part, parts), pn = part_cut(np, part + 1, parts) - ps;
        const int pn0 = __shfl_sync(0xffffffffu, pn, 0), pn1 = __shfl_sync(0xffffffffu, pn, 1);
        const int pn2 = __shfl_sync(0xffffffffu, pn, 2);
        const int lb = (p > 0 ? pn0 : 0) + (p > 1 ? pn1 : 0) + (p > 2 ? pn2 : 0);
        const int lo = max(lb, c0), hi = max(lo, min(lb + pn, c1));
        const int n = hi - lo, d = ps + (lo - lb);
        const int ntile = p == 0   ? (n + phase_tile_rows(0) - 1) / phase_tile_rows(0)
                          : p == 1 ? (n + phase_tile_rows(1) - 1) / phase_tile_rows(1)
                          : p == 2 ? (n + phase_tile_rows(2) - 1) / phase_tile_rows(2)
                                   : (n + phase_tile_rows(3) - 1) / phase_tile_rows(3);
        auto ptr_of = [](int x, int y) {
          return reinterpret_cast<const unsigned char*>((uintptr_t)(uint32_t)x | ((uintptr_t)(uint32_t)y << 32));
        };
        const int t0 = __shfl_sync(0xffffffffu, ntile, 0), t1 = __shfl_sync(0xffffffffu, ntile, 1);
        const int t2 = __shfl_sync(0xffffffffu, ntile, 2), t3 = __shfl_sync(0xffffffffu, ntile, 3);
        int t4 = 0;
        if (TAIL) {
          const TailGeom tg = tail_geom(pn0, pn1, pn2, __shfl_sync(0xffffffffu, pn, 3), c0, c1);
          t4 = tg.tiles;
          if (lane == 0) {
            G.lo[4] = tg.lo; G.hi[4] = tg.hi; G.first_tile[4] = t0 + t1 + t2 + t3;
            G.vrow[4] = tail_row(ta.new_v, tg.d); G.krow_tail = tail_row(ta.new_k, tg.d);
          }
        }
        if (lane < 4) {
          G.lo[p] = lo; G.hi[p] = hi;
          G.first_tile[p] = p == 0 ? 0 : p == 1 ? t0 : p == 2 ? t0 + t1 : t0 + t1 + t2;
          G.krow[p] = p < 3 ? (int64_t)a0.x + d : (int64_t)h2.y + d;
          G.k2[p] = ptr_of(a1.x, a1.y) + (int64_t)d * kq.sub2;
          G.k4[p] = ptr_of(a1.z, a1.w) + (int64_t)d * kq.sub4;
          G.k8[p] = ptr_of(a2.x, a2.y) + (int64_t)d * kq.n8;
          G.vrow[p] = ptr_of(a2.z, a2.w) + (int64_t)d * phase_row_bytes(p);
          G.vrow_idx[p] = a0.z >= 0 ? a0.z + d : -1;
          if (p < 3) { G.sc[p] = ptr_of(a3.x, a3.y) + 2 * d; G.zp[p] = ptr_of(a3.z, a3.w) + 2 * d; }
        }
        if (lane == 0) {
          G.vmaps = ptr_of(h2.z, h2.w);
          G.fast = 1;
          G.first_tile[NPH] = fits_q ? t0 + t1 + t2 + t3 + t4 : -1;
        }
        __threadfence_block();
        __syncwarp();
        bar_arrive(BAR_GEOM, CTA_THREADS);
        geom_done = true;
      }
    }
    if (!geom_done) bar_sync(BAR_VIEW, CTA_THREADS);       // the general path reads the view record
  } else {
    {
      const int* src = reinterpret_cast<const int*>(views + view_idx);
      int* dst = reinterpret_cast<int*>(&v);
      for (int i = tid; i < (int)(sizeof(rdkv_layer_view) / 4); i += FW * 32) dst[i] = ldg_keep(src + i);
    }
    if (prepared && MODE != MODE_WEIGHTS) {
      const int4* kp = reinterpret_cast<const int4*>(kslots + unit * nkb_max * 32 + lane);
      if (warp < nkb_max) { const int4 t = ldg_keep4(kp + warp * 32); km0 = {(uint32_t)t.x, (uint32_t)t.y, (uint32_t)t.z, (uint32_t)t.w}; }
      if (warp + FW < nkb_max) { const int4 t = ldg_keep4(kp + (warp + FW) * 32); km1 = {(uint32_t)t.x, (uint32_t)t.y, (uint32_t)t.z, (uint32_t)t.w}; }
    }
    if (MODE != MODE_WEIGHTS) {
      const int64_t q0 = ((int64_t)view_idx * H_q + hq0) * D;
      const int n = gcnt * D;
      if (q_dtype == RDKV_F32) {
        const float* qp = reinterpret_cast<const float*>(q) + q0;
        if ((reinterpret_cast<uintptr_t>(qp) & 15) == 0) {
          for (int i = 4 * tid; i < n; i += 4 * FW * 32) *reinterpret_cast<float4*>(f_q + i) = *reinterpret_cast<const float4*>(qp + i);
        } else {
          for (int i = tid; i < n; i += FW * 32) f_q[i] = qp[i];
        }
      } else {
        const uint16_t* qp = reinterpret_cast<const uint16_t*>(q) + q0;
        const bool bf = q_dtype == RDKV_BF16;
        auto cvt = [&](uint16_t x) { return bf ? __uint_as_float((uint32_t)x << 16) : h2f(x); };
        if ((reinterpret_cast<uintptr_t>(qp) & 7) == 0) {
          for (int i = 4 * tid; i < n; i += 4 * FW * 32) {
            const uint2 w = *reinterpret_cast<const uint2*>(qp + i);
            *reinterpret_cast<float4*>(f_q + i) = make_float4(cvt((uint16_t)w.x), cvt((uint16_t)(w.x >> 16)),
                                                              cvt((uint16_t)w.y), cvt((uint16_t)(w.y >> 16)));
          }
        } else {
          for (int i = tid; i < n; i += FW * 32) f_q[i] = cvt(qp[i]);
        }
      }
    }
    bar_sync(BAR_VIEW, CTA_THREADS);
  }
  if (!geom_done) { n2p = v.n_ch2_pad; n4p = v.n_ch4_pad; n8c = v.n_ch8; }

  // where this CTA's result goes: chunked units write one record per chunk (merged by the last
  // CTA of the unit to finish when the launch brings arrival counters, else by the combine kernel);
  // a whole unit writes the normalised result or one un-normalised record
  float* rec_base = (n_chunks > 1 || merged == nullptr) ? partials : merged;
  float* rec0 = rec_base != nullptr
                    ? rec_base + ((int64_t)(view_idx * H_q + hq0) * n_chunks + chunk) * RDKV_PARTIAL_STRIDE
                    : nullptr;
  const int64_t rec_stride = (int64_t)n_chunks * RDKV_PARTIAL_STRIDE;
  const bool direct = (n_chunks == 1 && out != nullptr);
  if (tid == 0) {
    s_epi.out_rows = out != nullptr ? out + ((int64_t)view_idx * H_q + hq0) * D : nullptr;
    s_epi.rec0 = rec0; s_epi.rec_stride = rec_stride; s_epi.row0 = (int64_t)view_idx * H_q + hq0;
    s_epi.how = MODE == MODE_WEIGHTS ? 2 : direct ? 1 : 0;
    s_epi.gcnt = gcnt; s_epi.n_chunks = n_chunks; s_epi.unit_y = unit_y;
  }

  const KDims kd = k_dims(n2p, n4p, n8c);
  const int d_pad = kd.n2p + kd.n4p + kd.n8;
  const StageLayout SL = stage_layout(kd.sub2, kd.sub4, kd.n8);
  const bool fits = SL.total <= stage_bytes && d_pad > 0 && d_pad <= DPAD_MAX && kd.nkb <= KB_MAX;   // view fits this launch

  // ── geometry, general path (staging warp, one lane per phase): live rows of this head are
  //    [0,n2) 2-bit, [n2,n2+n4) 4-bit, [..,t_v) 8-bit, [t_v, t_v+n16) fp16; the chunk takes
  //    [row_begin + chunk*chunk_rows, +chunk_rows) of them, cut at row_end.  The compute warps
  //    fold the queries meanwhile. ──
  if (warp == FW && !geom_done) {
    const HeadCounts hc = head_counts(v, h);
    const int p = lane & 3;
    const int c0 = row_begin + chunk * chunk_rows, c1 = n_chunks == 1 ? row_end : min(c0 + chunk_rows, row_end);
    // (MODE_SCORES: every stripe row below t_eff is scored, as one run of rows; the rows that
    //  belong to no token hold the zero point and score 0, as in the reference)
    const int b_lo = MODE == MODE_SCORES ? 0 : p == 0 ? 0 : p == 1 ? hc.n2 : p == 2 ? hc.n2 + hc.n4 : hc.t_v;
    const int b_hi = MODE == MODE_SCORES ? (p == 0 ? t_eff : 0)
                                         : p == 0 ? hc.n2 : p == 1 ? hc.n2 + hc.n4 : p == 2 ? hc.t_v : hc.t_v + hc.n16;
    // this part's share of the phase, then the chunk's window of the part's rows (numbered phase
    // after phase); lo, hi: the rows of the head it comes to
    const int np = b_hi - b_lo, ps = part_cut(np, part, parts), pn = part_cut(np, part + 1, parts) - ps;
    const int pn0 = __shfl_sync(0xffffffffu, pn, 0), pn1 = __shfl_sync(0xffffffffu, pn, 1);
    const int pn2 = __shfl_sync(0xffffffffu, pn, 2);
    const int lb = (p > 0 ? pn0 : 0) + (p > 1 ? pn1 : 0) + (p > 2 ? pn2 : 0);
    const int wl = max(lb, c0), wh = max(wl, min(lb + pn, c1));
    const int lo = b_lo + ps + (wl - lb);
    const int hi = lo + (wh - wl);
    const int n = hi - lo;
    const int ntile = (n + phase_tile_rows(p) - 1) / phase_tile_rows(p);
    const int64_t krow = (p < 3 || MODE == MODE_SCORES) ? lo : (int64_t)v.max_t_v + (lo - hc.t_v);   // stripe row
    const unsigned char* v16b = reinterpret_cast<const unsigned char*>(v.v16);
    const unsigned char* scb = reinterpret_cast<const unsigned char*>(v.v_scale);
    const unsigned char* zpb = reinterpret_cast<const unsigned char*>(v.v_zp);
    const unsigned char* gk2 = kd.sub2 ? v.k2 + h * v.k2_head_stride + krow * kd.sub2 : nullptr;
    const unsigned char* gk4 = kd.sub4 ? v.k4 + h * v.k4_head_stride + krow * kd.sub4 : nullptr;
    const unsigned char* gk8 = kd.n8 ? v.k8 + h * v.k8_head_stride + krow * kd.n8 : nullptr;
    const unsigned char* vlo = p == 0 ? v.v2 : p == 1 ? v.v4 : p == 2 ? v.v8 : v16b;
    const int64_t vext = p == 0 ? v.v2_bytes : p == 1 ? v.v4_bytes : p == 2 ? v.v8_bytes : v.v16_bytes;
    const int64_t vhs = p == 0 ? v.v2_head_stride : p == 1 ? v.v4_head_stride : p == 2 ? v.v8_head_stride
                                                                                     : 2 * v.v16_head_stride;
    const unsigned char* vb = vlo + h * vhs + (int64_t)(lo - b_lo) * phase_row_bytes(p);
    const unsigned char* gsc = scb + (h * v.v_meta_head_stride + lo) * 2;
    const unsigned char* gzp = zpb + (h * v.v_meta_head_stride + lo) * 2;
    bool fast = true;
    if (n > 0) {
      if (kd.sub2) fast = fast && blocks_inside(gk2, gk2 + (int64_t)n * kd.sub2, v.k2, v.k2 + v.k2_bytes);
      if (kd.sub4) fast = fast && blocks_inside(gk4, gk4 + (int64_t)n * kd.sub4, v.k4, v.k4 + v.k4_bytes);
      if (kd.n8) fast = fast && blocks_inside(gk8, gk8 + (int64_t)n * kd.n8, v.k8, v.k8 + v.k8_bytes);
      if (MODE != MODE_SCORES) fast = fast && blocks_inside(vb, vb + (int64_t)n * phase_row_bytes(p), vlo, vlo + vext);
      if (p < 3 && MODE != MODE_SCORES) {
        fast = fast && blocks_inside(gsc, gsc + n * 2, scb, scb + v.v_meta_bytes);
        fast = fast && blocks_inside(gzp, gzp + n * 2, zpb, zpb + v.v_meta_bytes);
      }
    }
    fast = __all_sync(0xffffffffu, fast);                  // lanes 4.. repeat lanes 0..3
    const int t0 = __shfl_sync(0xffffffffu, ntile, 0), t1 = __shfl_sync(0xffffffffu, ntile, 1);
    const int t2 = __shfl_sync(0xffffffffu, ntile, 2), t3 = __shfl_sync(0xffffffffu, ntile, 3);
    int t4 = 0;
    if (TAIL) {
      const TailGeom tg = tail_geom(pn0, pn1, pn2, __shfl_sync(0xffffffffu, pn, 3), c0, c1);
      t4 = tg.tiles;
      if (lane == 0) {
        G.lo[4] = tg.lo; G.hi[4] = tg.hi; G.first_tile[4] = t0 + t1 + t2 + t3;
        G.vrow[4] = tail_row(ta.new_v, tg.d); G.krow_tail = tail_row(ta.new_k, tg.d);
      }
    }
    if (lane < 4) {
      G.lo[p] = lo; G.hi[p] = hi;
      G.first_tile[p] = p == 0 ? 0 : p == 1 ? t0 : p == 2 ? t0 + t1 : t0 + t1 + t2;
      G.krow[p] = krow;
      G.k2[p] = gk2; G.k4[p] = gk4; G.k8[p] = gk8; G.vrow[p] = vb;
      G.vrow_idx[p] = -1;
      if (p < 3) { G.sc[p] = gsc; G.zp[p] = gzp; }
    }
    if (lane == 0) {
      G.vmaps = nullptr;
      G.fast = fast ? 1 : 0;
      G.first_tile[NPH] = (!fits || (MODE != MODE_SCORES && hc.n16 > 0 && v.v16 == nullptr)) ? -1 : t0 + t1 + t2 + t3 + t4;
    }
    __threadfence_block();
    __syncwarp();
    bar_arrive(BAR_GEOM, CTA_THREADS);
  }

  // ── q*scale in MMA fragment order and the zero-point bias (compute warps, while the staging
  //    warp works out the geometry and starts the first copies).  The head's scales, zero points
  //    and channel permutation come into shared memory with one coalesced read each; the fold
  //    itself then gathers from shared memory only. ──
  // ── tail mode: rotary embedding of the query rows, the queries as fragments of the tail's score
  //    product, and the token being decoded (its key row rotated, scored, appended to the tail) ──
  uint2* qtA = reinterpret_cast<uint2*>(tail + tail_bytes);                  // [8][32]
  float* f_kc = reinterpret_cast<float*>(tail + tail_bytes + TAILQ_BYTES);   // [128] new key row (rotated, rounded to the tail's type)
  float* f_vc = f_kc + D;                                                    // [128] new value row
  float* s_cur = f_vc + D;                                                   // [GH] the new token's scores, base-2 units
  const bool seeded = TAIL && ta.k_cur != nullptr && chunk == 0 && part == 0;
  if (TAIL && warp < FW) {
    const bool rope = ta.rope_cos != nullptr;
    float rc = 1.f, rs = 0.f;                              // every pair a thread rotates has the same position tid & 63
    if (rope) {
      const int64_t e = (int64_t)view_idx * ta.rope_view_stride + (tid & 63);
      rc = load_q(ta.rope_cos, ta.rope_dtype, e); rs = load_q(ta.rope_sin, ta.rope_dtype, e);
    }
    auto round_as = [](float x, int dt) {
      return dt == RDKV_F16 ? __half2float(__float2half_rn(x)) : dt == RDKV_BF16 ? __bfloat162float(__float2bfloat16_rn(x)) : x;
    };
    // half format: (x[i], x[i+64]) -> (x[i] c - x[i+64] s, x[i+64] c + x[i] s); products and sums rounded
    // one by one, the result rounded to the tensor's own type (as the in-place operation would leave it)
    auto rotate = [&](float& lo, float& hi, int dt) {
      const float a = __fsub_rn(__fmul_rn(lo, rc), __fmul_rn(hi, rs)), b = __fadd_rn(__fmul_rn(hi, rc), __fmul_rn(lo, rs));
      lo = round_as(a, dt); hi = round_as(b, dt);
    };
    if (rope && fits) {
      for (int idx = tid; idx < gcnt * 64; idx += FW * 32) {
        float* row = f_q + (idx >> 6) * D + (idx & 63);
        float lo = row[0], hi = row[64];
        rotate(lo, hi, q_dtype);
        row[0] = lo; row[64] = hi;
      }
    }
    if (seeded) {
      const int64_t e = ((int64_t)view_idx * (H_q / g) + h) * D;
      if (tid < 64) {
        float lo = load_q(ta.k_cur, ta.dtype, e + tid), hi = load_q(ta.k_cur, ta.dtype, e + tid + 64);
        if (rope) rotate(lo, hi, ta.dtype);
        f_kc[tid] = lo; f_kc[tid + 64] = hi;
      } else {
        const int i = 2 * (tid - 64);
        f_vc[i] = load_q(ta.v_cur, ta.dtype, e + i); f_vc[i + 1] = load_q(ta.v_cur, ta.dtype, e + i + 1);
      }
    }
    bar_sync(BAR_COMPUTE, FW * 32);                        // rotated rows are in shared memory
    // B fragments of the tail's score product: MMA m of a 16-row group contracts channels
    // 32*(m/2) + 8j + 4*(m%2) + {0,1 | 2,3} of thread j against the K words the thread loads
    for (int m = warp; m < 8; m += FW) {
      const bool ok = r < gcnt;
      const float* row = f_q + (ok ? r : 0) * D + 32 * (m >> 1) + 8 * j + 4 * (m & 1);
      qtA[m * 32 + lane] = ok ? make_uint2(pack_h2(row[0], row[1]), pack_h2(row[2], row[3])) : make_uint2(0u, 0u);
    }
    if (seeded) {
      for (int hh = 2 * warp; hh < 2 * warp + 2; ++hh) {   // the new token's scores: warp w takes heads 2w, 2w+1
        float a = 0.f;
        if (hh < gcnt)
          for (int c = lane; c < D; c += 32) a = fmaf(f_q[hh * D + c], f_kc[c], a);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0) s_cur[hh] = a * (INV_SQRT_D * LOG2E);
      }
      if (ta.append && hgrp == 0) {                        // the rotated key row and the value row become tail row n_tail
        if (n_tail < ta.cap) {
          uint16_t* kd_row = reinterpret_cast<uint16_t*>(const_cast<unsigned char*>(tail_row(ta.new_k, n_tail)));
          uint16_t* vd_row = reinterpret_cast<uint16_t*>(const_cast<unsigned char*>(tail_row(ta.new_v, n_tail)));
          const bool bf = ta.dtype == RDKV_BF16;
          auto bits = [&](float x) {
            return bf ? __bfloat16_as_ushort(__float2bfloat16_rn(x)) : __half_as_ushort(__float2half_rn(x));
          };
          kd_row[tid] = bits(f_kc[tid]); vd_row[tid] = bits(f_vc[tid]);
        } else if (tid == 0 && status != nullptr) {
          atomicOr(status, 4);
        }
      }
    }
  }

  if (MODE != MODE_WEIGHTS && warp < FW && fits && prepared) {
    // prepared table: this thread's slot quadruples were requested at entry, together with the
    // view record; nothing else comes from global memory.  Blocks warp and warp + FW are folded
    // side by side (independent chains), any further ones in a loop.
    const bool head_ok = r < gcnt;
    const float* qrow = f_q + (head_ok ? r : 0) * D;
    float bias_part = 0.f;
    auto fold_block = [&](const KSlotRec& km, int kb, float& bias) {
      const int ex2b = kb < 2 * kd.nsp2 ? 4 * (kb & 1) : 0;            // exponent of the factor of e = 0, 1
      const int exs = kb < 2 * kd.nsp2 ? 2 : kb < 2 * kd.nsp2 + 2 * kd.nsp4 ? 4 : 0;   // added for e = 2, 3
      float val[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ex = ex2b + (e >> 1) * exs;
        const float scv = h2f((uint16_t)((e < 2 ? km.sc01 : km.sc23) >> (16 * (e & 1))));
        const float zpv = (float)((km.zp4 >> (8 * e)) & 255u);
        float x = __half2float(__float2half_rn(qrow[(km.perm4 >> (8 * e)) & 127u] * scv * pow2i(-ex)));
        if (!head_ok) x = 0.f;
        bias += zpv * (x * pow2i(ex));
        val[e] = x;
      }
      qsA[kb * 32 + lane] = make_uint2(pack_h2(val[0], val[1]), pack_h2(val[2], val[3]));
    };
    // (one copy of the fold code: it runs once per CTA, from a cold instruction cache.  The first
    // two blocks of a warp are summed on their own and then added, further blocks term by term.)
    int nb = 0;
#pragma unroll 1
    for (int kb = warp; kb < kd.nkb; kb += FW, ++nb) {
      KSlotRec km = nb == 0 ? km0 : km1;
      if (nb >= 2) {
        const int4 t = *(reinterpret_cast<const int4*>(kslots + unit * nkb_max * 32 + lane) + kb * 32);
        km = {(uint32_t)t.x, (uint32_t)t.y, (uint32_t)t.z, (uint32_t)t.w};
      }
      float b = nb < 2 ? 0.f : bias_part;
      fold_block(km, kb, b);
      bias_part = nb < 2 ? bias_part + b : b;
    }
    bias_part += __shfl_xor_sync(0xffffffffu, bias_part, 1);
    bias_part += __shfl_xor_sync(0xffffffffu, bias_part, 2);
    if (j == 0) s_bias[warp][r] = bias_part;             // summed over the warps where it is used
    bar_sync(BAR_COMPUTE, FW * 32);
  } else if (MODE != MODE_WEIGHTS && warp < FW && fits) {
    {
      const uint16_t* sc = v.k_scale + (int64_t)h * d_pad;
      const uint16_t* zp = v.k_zp + (int64_t)h * d_pad;
      const int64_t* perm = v.k_perm + (int64_t)h * v.k_perm_head_stride;
      for (int i = tid; i < d_pad; i += FW * 32) {
        f_sc[i] = sc[i]; f_zp[i] = zp[i]; f_pm[i] = (uint16_t)(perm[i] & (D - 1));
      }
    }
    bar_sync(BAR_COMPUTE, FW * 32);
    const bool head_ok = r < gcnt;
    const float* qrow = f_q + (head_ok ? r : 0) * D;
    float bias_part = 0.f;                                 // thread (r = head, j) sums its own slots
#pragma unroll 1
    for (int kb = warp; kb < kd.nkb; kb += FW) {
      float val[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float f;
        const int slot = k_slot(kd, kb, j, e, &f);
        float x = 0.f;
        if (slot >= 0 && head_ok) {
          x = __half2float(__float2half_rn(qrow[f_pm[slot]] * h2f(f_sc[slot]) / f));
          bias_part += h2f(f_zp[slot]) * (x * f);
        }
        val[e] = x;
      }
      qsA[kb * 32 + lane] = make_uint2(pack_h2(val[0], val[1]), pack_h2(val[2], val[3]));
    }
    bias_part += __shfl_xor_sync(0xffffffffu, bias_part, 1);
    bias_part += __shfl_xor_sync(0xffffffffu, bias_part, 2);
    if (j == 0) s_bias[warp][r] = bias_part;             // summed over the warps where it is used
    bar_sync(BAR_COMPUTE, FW * 32);
  }
  if (warp < FW) bar_sync(BAR_GEOM, CTA_THREADS);          // geometry published
  const int total_tiles = G.first_tile[NPH];

  if (total_tiles < 0 || (total_tiles == 0 && !seeded)) {  // nothing live here: empty records
    if (total_tiles < 0 && tid == 0 && status != nullptr) atomicOr(status, 2);
    if (MODE == MODE_SCORES) return;
    if (direct) {
      for (int i = tid; i < gcnt * D; i += blockDim.x) out[((int64_t)view_idx * H_q + hq0) * D + i] = 0.f;
    } else {
      for (int i = tid; i < gcnt * RDKV_PARTIAL_STRIDE; i += blockDim.x) {
        const int hq = i / RDKV_PARTIAL_STRIDE, e = i % RDKV_PARTIAL_STRIDE;
        rec0[hq * rec_stride + e] = (e == 0) ? -INFINITY : 0.f;
      }
    }
    if (ATTN && n_chunks > 1 && unit_ctr != nullptr)
      chunk_merge<false>(partials, unit_ctr + unit_y, n_chunks, gcnt,
                         (int64_t)view_idx * H_q + hq0, out, merged);
    return;
  }

  if (warp == FW) {
    // ── staging warp ──────────────────────────────────────────────────────────
    // Tiles are planned 32 at a time, one per lane (where each of a tile's six byte ranges
    // starts, how long it is, where it goes), so that the per-tile work is a table look-up and
    // the copy instructions.  The warp only ever waits for a free slot; a tile's landing is
    // signalled to the compute warps by the copies themselves (mbarrier transaction bytes on
    // the bulk-copy path, arrival on completion of the cp.async copies otherwise).
    const unsigned char* v16b = reinterpret_cast<const unsigned char*>(v.v16);
    const unsigned char* scb = reinterpret_cast<const unsigned char*>(v.v_scale);
    const unsigned char* zpb = reinterpret_cast<const unsigned char*>(v.v_zp);
    const bool fast = G.fast != 0;
    const uint64_t pol_stream = l2_policy_stream();
#pragma unroll 1
    for (int it = 0; it < total_tiles; ++it) {
      const int slot = it % PLAN_TILES;
      if (slot == 0) {                                     // plan tiles [it, it + 32)
        __syncwarp();
        if (it + lane < total_tiles) {
          const TileDesc t = tile_of<NPH>(G, it + lane);
          const int p = t.phase;
          TilePlan& P = s_plan[lane];
          if (TAIL && p == 4) {
            // tail tile: its V rows at the start of the V area, its K rows behind them; the block
            // goes to warp (tile number within the tail) % FW
            P.rg[0] = RangePlan{G.vrow[4] + (int64_t)t.row0 * 256, t.n * 256, (uint32_t)SL.v};
            P.rg[1] = RangePlan{G.krow_tail + (int64_t)t.row0 * 256, t.n * 256, (uint32_t)(SL.v + TAIL_TILE * 256)};
#pragma unroll
            for (int k = 2; k < 6; ++k) P.rg[k] = RangePlan{nullptr, 0, 0u};
            P.info.phase = 4 | ((t.row0 / TAIL_TILE) & (FW - 1)) << 8; P.info.n = t.n;
            P.info.offs = 0u; P.info.krow0 = 0;
          } else {
          const unsigned char* a_k2 = G.k2[p] + (int64_t)t.row0 * kd.sub2;
          const unsigned char* a_k4 = G.k4[p] + (int64_t)t.row0 * kd.sub4;
          const unsigned char* a_k8 = G.k8[p] + (int64_t)t.row0 * kd.n8;
          const unsigned char* a_v = G.vrow[p] + (int64_t)t.row0 * phase_row_bytes(p);
          const unsigned char* a_sc = G.sc[p < 3 ? p : 0] + t.row0 * 2;
          const unsigned char* a_zp = G.zp[p < 3 ? p : 0] + t.row0 * 2;
          // the V rows: one box of the phase's tensor map (src = the map, len = the box's bytes, dst_off = its
          // first row) when the table has maps, else copies by the lanes at the padded pitch
          // (a ragged last fp16 block goes that way too: the rows behind it are cleared)
          const bool v_any = MODE != MODE_SCORES && t.n > 0;
          const bool v_tma = v_any && p >= V_PAD_FROM && fast && G.vmaps != nullptr && G.vrow_idx[p] >= 0 && (p < 3 || (t.n & 31) == 0);
          if (v_tma) P.rg[0] = RangePlan{G.vmaps + 128 * p, phase_tile_rows(p) * phase_pitch(p), (uint32_t)(G.vrow_idx[p] + t.row0)};
          else P.rg[0] = RangePlan{a_v, v_any ? t.n * phase_row_bytes(p) : 0, (uint32_t)SL.v};
          P.rg[1] = RangePlan{a_k2, MODE == MODE_WEIGHTS ? 0 : t.n * kd.sub2, (uint32_t)SL.k2};
          P.rg[2] = RangePlan{a_k4, MODE == MODE_WEIGHTS ? 0 : t.n * kd.sub4, (uint32_t)SL.k4};
          P.rg[3] = RangePlan{a_k8, MODE == MODE_WEIGHTS ? 0 : t.n * kd.n8, (uint32_t)SL.k8};
          P.rg[4] = RangePlan{a_sc, (p < 3 && MODE != MODE_SCORES) ? t.n * 2 : 0, (uint32_t)SL.sc};
          P.rg[5] = RangePlan{a_zp, (p < 3 && MODE != MODE_SCORES) ? t.n * 2 : 0, (uint32_t)SL.zp};
          auto low4 = [](const unsigned char* x) { return (uint32_t)reinterpret_cast<uintptr_t>(x) & 15u; };
          int blocks_before = 0;                          // 32-row blocks of the chunk ahead of this tile: the tile's first block goes to warp (that % FW)
#pragma unroll
          for (int qq = 0; qq < 3; ++qq)
            if (qq < p) blocks_before += (G.hi[qq] - G.lo[qq] + 31) >> 5;
          blocks_before += t.row0 >> 5;
          P.info.phase = p | (blocks_before & (FW - 1)) << 8 | (v_tma ? 1 << 16 : (v_any && (p >= V_PAD_FROM || !fast || low4(a_v) != 0u)) ? 1 << 17 : 0); P.info.n = t.n;
          P.info.offs = low4(a_k2) | low4(a_k4) << 4 | low4(a_k8) << 8 |
                        (p < 3 ? low4(a_sc) << 16 | low4(a_zp) << 20 : 0u);
          P.info.krow0 = (int)(G.krow[p] + t.row0);
          }
        }
        __syncwarp();
      }
      // this tile's plan: lanes 0..5 take one range each (before the wait for the slot)
      const int stage = it % FSTAGES;
      RangePlan rp = s_plan[slot].rg[lane < 6 ? lane : 0];
      if (lane >= 6) rp.len = 0;
      const TileInfo ti = s_plan[slot].info;
      const bool v_tma = (ti.phase >> 16) & 1, v_lanes = (ti.phase >> 17) & 1;   // how the V rows travel (neither: the tail, or none)
      const uintptr_t a = reinterpret_cast<uintptr_t>(rp.src), a0 = a & ~(uintptr_t)15;
      uint32_t bytes = rp.len > 0 ? (uint32_t)(((a + rp.len + 15) & ~(uintptr_t)15) - a0) : 0u;   // covering 16-byte blocks
      if (lane == 0 && v_tma) bytes = (uint32_t)rp.len;    // (the whole box is counted, whatever part of it lies in the tensor)
      if (lane == 0 && v_lanes) bytes = 0u;
      uint32_t total = bytes;
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
      const uint32_t sbu = smem0 + stage * stage_bytes;

      if (it >= FSTAGES) bar_sync(BAR_FREE + stage, CTA_THREADS);          // compute warps left the slot
      if (fast) {
        // every range is contiguous in its tensor: ONE bulk copy each, completion counted in bytes
        if (lane == 0) mbar_expect_tx(&s_full[stage], total);
        __syncwarp();
        {
          const bool by_map = lane == 0 && v_tma;
          tma_g2s_2d_if(by_map, sbu + SL.v, rp.src, 0, (int)rp.dst_off, &s_full[stage], pol_stream);
#if RDKV_L2HINT
          bulk_g2s_hint_if(bytes != 0u && !by_map, sbu + rp.dst_off, reinterpret_cast<const void*>(a0), bytes, &s_full[stage], pol_stream);
#else
          if (bytes != 0u && !by_map) bulk_g2s(sbu + rp.dst_off, reinterpret_cast<const void*>(a0), bytes, &s_full[stage]);
#endif
        }
        if (v_lanes) {
          const RangePlan rv = s_plan[slot].rg[0];
          stage_v_rows_padded(smem_raw + (size_t)stage * stage_bytes + SL.v, rv.src, ti.n, phase_row_bytes(ti.phase & 7), phase_pitch(ti.phase & 7), lane);
        }
      } else {
        // a range whose covering blocks stick out of its tensor: guarded 16-byte copies by all lanes
        unsigned char* sb = smem_raw + (size_t)stage * stage_bytes;
        const int p = ti.phase & 7;
#pragma unroll 1
        for (int k = 0; k < 6; ++k) {
          const RangePlan rk = s_plan[slot].rg[k];
          if (rk.len <= 0) continue;
          if (TAIL && p == 4) {                            // tail rows are 16-byte aligned: nothing sticks out
            stage_range_guarded(sb + rk.dst_off, rk.src, rk.len, rk.src, rk.src + rk.len, lane, 32);
            continue;
          }
          if (k == 0) {                                    // V rows: at the padded pitch
            stage_v_rows_padded(sb + SL.v, rk.src, ti.n, phase_row_bytes(p), phase_pitch(p), lane);
            continue;
          }
          const unsigned char* lo = k == 0 ? (p == 0 ? v.v2 : p == 1 ? v.v4 : p == 2 ? v.v8 : v16b)
                                  : k == 1 ? v.k2 : k == 2 ? v.k4 : k == 3 ? v.k8 : k == 4 ? scb : zpb;
          const int64_t ext = k == 0 ? (p == 0 ? v.v2_bytes : p == 1 ? v.v4_bytes : p == 2 ? v.v8_bytes : v.v16_bytes)
                            : k == 1 ? v.k2_bytes : k == 2 ? v.k4_bytes : k == 3 ? v.k8_bytes : v.v_meta_bytes;
          stage_range_guarded(sb + rk.dst_off, rk.src, rk.len, lo, lo + ext, lane, 32);
        }
      }
      // rows past the tile's end must hold finite fp16 data in the fp16 phase: clear the
      // rest of the last 32-row block beyond the copied blocks
      if ((ti.phase & 7) >= 3 && (ti.n & 31)) {
        const int pitch = phase_pitch(ti.phase & 7);       // (the tail's rows: 256 bytes; fp16 V rows: padded)
        const int first = ti.n * pitch;
        const int last = min(((ti.n + 31) & ~31) * pitch, V_STAGE);
        unsigned char* sv = smem_raw + (size_t)stage * stage_bytes + SL.v;
        for (int i = first + 4 * lane; i < last; i += 4 * 32) *reinterpret_cast<uint32_t*>(sv + i) = 0u;
      }
      if (lane == 0) s_tile[stage] = ti;
      mbar_arrive_on_copies(&s_full[stage]);                               // fires when this lane's cp.async copies land
      mbar_arrive(&s_full[stage]);                                         // releases this lane's plain stores
    }
    cp_wait<0>();
  }

  // ── workers ─────────────────────────────────────────────────────────────────
  // Score product orientation: rows on M (16 per MMA), query heads on N.  Thread (r, j)
  // then holds scores of rows g16+r and g16+r+8 for heads 2j and 2j+1 — the same two
  // heads whose output columns it accumulates in the P.V product.
#include "decode_state.inc"
  // reference maxima of the tail's scores (they carry no zero-point bias): what cb holds beyond the bias
  float tref_e = he_ok ? 0.f : INFINITY, tref_o = ho_ok ? 0.f : INFINITY;
  if (TAIL && seeded && warp < FW) {
    // the token being decoded starts the running softmax: reference = its score, weight 1, value row
    // as the accumulator of warp 0
    if (he_ok) { m_e = s_cur[2 * j]; cb_e = b1e + m_e; thr_e = RESCALE_TH; tref_e = m_e; }
    if (ho_ok) { m_o = s_cur[2 * j + 1]; cb_o = b1o + m_o; thr_o = RESCALE_TH; tref_o = m_o; }
    if (warp == 0) {
      cur_phase = 3;
      if (r == 0) { l_e = he_ok ? 1.f : 0.f; l_o = ho_ok ? 1.f : 0.f; }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int ch = 4 * r + 2 * (i >> 2) + 32 * (i & 3);
        acc[i][0] = he_ok ? f_vc[ch] : 0.f; acc[i][1] = ho_ok ? f_vc[ch] : 0.f;
        acc[i][2] = he_ok ? f_vc[ch + 1] : 0.f; acc[i][3] = ho_ok ? f_vc[ch + 1] : 0.f;
      }
    }
  }
  const uint32_t qt_lane = smem_u32(qtA) + 8 * lane;
  const bool tail_bf = TAIL && ta.dtype == RDKV_BF16;

#pragma unroll 1
  for (int it = 0; warp < FW && it < total_tiles; ++it) {
    const int stage = it % FSTAGES;
    {                                                      // wait (bounded) until the tile in this slot has landed
      const uint32_t parity = (it / FSTAGES) & 1;
      unsigned spins = 0;
      while (!mbar_try_wait(&s_full[stage], parity)) {
        if (++spins > WAIT_LIMIT) {                        // give up: flag it and go on (results are then invalid)
          if (lane == 0 && status != nullptr) atomicOr(status, 1);
          break;
        }
      }
    }
    const TileInfo t = s_tile[stage];
    const int p = t.phase & 7;
    // this warp takes the tile's 32-row blocks pb, pb+FW, ... (two 16-row MMA groups each, worked on
    // together so that the two dependency chains overlap); the start rotates from tile to tile so
    // that short tiles (fewer blocks than warps) do not always land on the same warps
    const int nblocks = (t.n + 31) >> 5;
    const int pb = (TAIL && p == 4) ? (warp + FW - ((t.phase >> 8) & (FW - 1))) % FW
                                    : (warp + FW - (it * (TILE_MAX / 128)) % FW) % FW;

#include "decode_tile.inc"
    if (it + FSTAGES < total_tiles) bar_arrive(BAR_FREE + stage, CTA_THREADS);   // slot may be refilled
  }

  if (MODE == MODE_SCORES) return;
  // ── merge the four workers and write the chunk's record ─────────────────────
  if (cur_phase >= 0) {                                    // accumulators to true units
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = pow2i(acc_exp(cur_phase, i & 3));
      acc[i][0] *= f; acc[i][1] *= f; acc[i][2] *= f; acc[i][3] *= f;
    }
  }
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {                       // rows are spread over r: lanes 4r + j
    l_e += __shfl_xor_sync(0xffffffffu, l_e, o); l_o += __shfl_xor_sync(0xffffffffu, l_o, o);
  }
  __syncthreads();                                         // every worker is done with its stages
  float* red = reinterpret_cast<float*>(smem_raw);         // [FW][GH][128]
  if (warp < FW && r == 0) {
    s_ml[warp][2 * j][0] = m_e; s_ml[warp][2 * j][1] = l_e; s_ml[warp][2 * j][2] = zacc[0];
    s_ml[warp][2 * j + 1][0] = m_o; s_ml[warp][2 * j + 1][1] = l_o; s_ml[warp][2 * j + 1][2] = zacc[1];
  }
#pragma unroll
  for (int i = 0; i < 8 && warp < FW; ++i) {
    const int ch = 4 * r + 2 * (i >> 2) + 32 * (i & 3);
    float* o0 = red + ((warp * GH + 2 * j) * D);
    float* o1 = o0 + D;
    o0[ch] = acc[i][0]; o1[ch] = acc[i][1]; o0[ch + 1] = acc[i][2]; o1[ch + 1] = acc[i][3];
  }
  __syncthreads();
  const EpiInfo ep = s_epi;
  final_merge<false>(red, &s_ml[0][0][0], ep.gcnt, ep.how, ep.out_rows, ep.rec0, ep.rec_stride);
  if (ATTN && ep.n_chunks > 1 && unit_ctr != nullptr)
    chunk_merge<false>(partials, unit_ctr + ep.unit_y, ep.n_chunks, ep.gcnt, ep.row0, out, merged);
}


// ── persistent form ──────────────────────────────────────────────────────────
// The same work with ONE resident CTA per slot that goes through work items item, item + grid, ...
// (the item order of decode_fused_kernel: whole units first, then chunks).  The staging warp
// runs ahead of the compute warps across item boundaries — while they merge an item and fold the
// next item's queries, its first tiles are already on their way — so the round trips of a CTA's
// start (unit record, first tile) and the drain of its pipeline are paid once per CTA, not once
// per item.  Needs a prepared table whose units all lie on whole 16-byte blocks, no mask, 16-byte
// aligned queries.
//   * ring slots are handed back through mbarriers (s_empty: one arrival per compute warp), so the
//     staging warp needs no knowledge of the compute warps' position; every wait is bounded;
//   * an item's first tile brings the item's header along on the same mbarrier: its raw query rows
//     and its K slot table (two header buffers, alternating), and the staging warp publishes the
//     item's dimensions next to the tile's descriptor; an item without live rows gets an empty tile;
//   * the compute warps merge in the ring slot of the item's last tile and hand that slot back only
//     after the merge.
//   * items are handed out dynamically: a CTA starts with item blockIdx.x and draws every further one
//     from a counter in global memory (work[0]) when its staging warp has sent the current item's
//     last tile — the compute warps are two tiles behind, which hides the round trip; the last CTA
//     to run dry puts the counters (work[0], work[1]) back to zero for the next launch.
struct ItemInfo { int n2p, n4p, n8c, total, item, pad0, pad1, pad2; };

template <int MODE>
__global__ void __launch_bounds__(CTA_THREADS, RDKV_MINB)
decode_persist_kernel(const void* __restrict__ q, int q_dtype, int H_q, int g, int chunk_rows, int k_chunks,
                      int n_whole, int n_items, int stage_bytes, float* __restrict__ partials,
                      float* __restrict__ out, int* __restrict__ status, const UnitRec* __restrict__ unit_recs,
                      const KSlotRec* __restrict__ kslots, int nkb_max, int* __restrict__ unit_ctr,
                      float* __restrict__ merged, int row_begin, int row_end, int part, int parts,
                      int* __restrict__ work) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ CtaGeom G;                            // private to the staging warp
  __shared__ float s_ml[FW][GH][3];
  __shared__ float s_bias[FW][GH];                 // (not in s_ml: a warp may fold the next item while others still merge this one)
  __shared__ EpiInfo s_epi;
  __shared__ TileInfo s_tile[FSTAGES];
  __shared__ ItemInfo s_item[2];
  __shared__ TilePlan s_plan[PLAN_TILES];
  __shared__ __align__(8) uint64_t s_full[FSTAGES];    // tile in slot s has landed
  __shared__ __align__(8) uint64_t s_empty[FSTAGES];   // the compute warps are done with slot s

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r = lane >> 2, j = lane & 3;
  const int n_hgrp = (g + GH - 1) / GH;
  const int hy = (H_q / g) * n_hgrp;
  const uint32_t smem0 = smem_u32(smem_raw);
  const uint32_t qs_base = smem0 + FSTAGES * stage_bytes;  // uint2 qsA[nkb][32]
  unsigned char* tail = smem_raw + (size_t)FSTAGES * stage_bytes;
  uint2* qsA = reinterpret_cast<uint2*>(tail);
  const int q_elt = q_dtype == RDKV_F32 ? 4 : 2;
  const int hdr_q_bytes = GH * D * q_elt;                  // raw query rows of an item
  const int hdr_bytes = hdr_q_bytes + nkb_max * 32 * (int)sizeof(KSlotRec);
  unsigned char* hdr0 = tail + nkb_max * 256;
  constexpr int BAR_COMPUTE = 1 + FSTAGES;
  const struct { const float* mask; int64_t mask_row_stride; } v = {nullptr, 0};   // (no mask in this form)
  float* const aux = nullptr;
  const int64_t aux_stride = 0;
  const int t_eff = 0;

  if (warp == FW) {
    if (lane < FSTAGES) { mbar_init(&s_full[lane], 64); mbar_init(&s_empty[lane], FW); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

#if RDKV_STATIC_ROUNDS
#ifndef RDKV_DYN_TAIL
#define RDKV_DYN_TAIL 2
#endif
  const int static_rounds = max(1, n_items / (int)gridDim.x - RDKV_DYN_TAIL);
#endif
  int git = 0;                                             // tiles this CTA has been through (empty items count one)
  int li = 0;                                              // items this CTA has been through
  int item = blockIdx.x;                                   // staging warp: the item in hand; compute warps: as told with its first tile
#pragma unroll 1
  for (;; ++li) {
    int next_item = 0;
    if (warp == FW) {
      if (item >= n_items) {                               // nothing left: tell the compute warps (an empty tile without an item) and leave
        const int stage = git % FSTAGES;
        if (git >= FSTAGES) {
          const uint32_t parity = ((git / FSTAGES) - 1) & 1;
          unsigned spins = 0;
          while (!mbar_try_wait(&s_empty[stage], parity)) {
            if (++spins > WAIT_LIMIT) {
              if (lane == 0 && status != nullptr) atomicOr(status, 1);
              break;
            }
          }
        }
        if (lane == 0) {
          s_tile[stage] = TileInfo{0, 0, 0u, 0};
          s_item[li & 1] = ItemInfo{0, 0, 0, 0, -1, 0, 0, 0};
          const int done = atomicAdd(work + 1, 1);         // the last CTA to run dry resets the counters
          if (done == (int)gridDim.x - 1) { work[0] = 0; work[1] = 0; }
        }
        mbar_arrive_on_copies(&s_full[stage]);
        mbar_arrive(&s_full[stage]);
        break;
      }
    } else {
      // compute warps: the item comes with its first tile
      const int st = git % FSTAGES;
      const uint32_t parity = (git / FSTAGES) & 1;
      unsigned spins = 0;
      while (!mbar_try_wait(&s_full[st], parity)) {
        if (++spins > WAIT_LIMIT) {
          if (lane == 0 && status != nullptr) atomicOr(status, 1);
          break;
        }
      }
      item = s_item[li & 1].item;
      if (item < 0 || item >= n_items) break;
    }
    int unit_y, chunk, n_chunks;
    if (item < n_whole) {
      unit_y = item; chunk = 0; n_chunks = 1;
    } else {
      const int jj = item - n_whole;
      unit_y = n_whole + jj / k_chunks; chunk = jj % k_chunks; n_chunks = k_chunks;
    }
    const int view_idx = unit_y / hy;
    const int h = (unit_y % hy) / n_hgrp, hgrp = (unit_y % hy) % n_hgrp;
    const int gh0 = hgrp * GH, gcnt = min(GH, g - gh0);
    const int hq0 = h * g + gh0;
    const int64_t unit = (int64_t)view_idx * (H_q / g) + h;
    unsigned char* hdr = hdr0 + (li & 1) * hdr_bytes;

    if (warp == FW) {
      // ── staging warp: geometry of the item from its unit record, then its tiles ──
      const int4* up = reinterpret_cast<const int4*>(unit_recs + unit);
      const int p = lane & 3;
      const int4 h1 = ldg_keep4(up + 1), h2 = ldg_keep4(up + 2);
      const int4 a0 = ldg_keep4(up + 3 + 4 * p), a1 = ldg_keep4(up + 4 + 4 * p), a2 = ldg_keep4(up + 5 + 4 * p),
                 a3 = ldg_keep4(up + 6 + 4 * p);
      const int n2p = h1.z, n4p = h1.w, n8c = h2.x;
      const KDims kd = k_dims(n2p, n4p, n8c);
      const StageLayout SL = stage_layout(kd.sub2, kd.sub4, kd.n8);
      const bool fits = (h1.x & 3) == 3 && SL.total <= stage_bytes && kd.n2p + kd.n4p + kd.n8 > 0 &&
                        kd.n2p + kd.n4p + kd.n8 <= DPAD_MAX && kd.nkb <= KB_MAX && kd.nkb <= nkb_max;
      const int c0 = row_begin + chunk * chunk_rows, c1 = n_chunks == 1 ? row_end : min(c0 + chunk_rows, row_end);
      const int np = a0.y - a0.x, ps = part_cut(np, part, parts), pn = part_cut(np, part + 1, parts) - ps;
      const int pn0 = __shfl_sync(0xffffffffu, pn, 0), pn1 = __shfl_sync(0xffffffffu, pn, 1);
      const int pn2 = __shfl_sync(0xffffffffu, pn, 2);
      const int lb = (p > 0 ? pn0 : 0) + (p > 1 ? pn1 : 0) + (p > 2 ? pn2 : 0);
      const int lo = max(lb, c0), hi = max(lo, min(lb + pn, c1));
      const int n = hi - lo, d = ps + (lo - lb);
      const int ntile = p == 0   ? (n + phase_tile_rows(0) - 1) / phase_tile_rows(0)
                        : p == 1 ? (n + phase_tile_rows(1) - 1) / phase_tile_rows(1)
                        : p == 2 ? (n + phase_tile_rows(2) - 1) / phase_tile_rows(2)
                                 : (n + phase_tile_rows(3) - 1) / phase_tile_rows(3);
      auto ptr_of = [](int x, int y) {
        return reinterpret_cast<const unsigned char*>((uintptr_t)(uint32_t)x | ((uintptr_t)(uint32_t)y << 32));
      };
      const int t0 = __shfl_sync(0xffffffffu, ntile, 0), t1 = __shfl_sync(0xffffffffu, ntile, 1);
      const int t2 = __shfl_sync(0xffffffffu, ntile, 2), t3 = __shfl_sync(0xffffffffu, ntile, 3);
      __syncwarp();                                        // (the plan of the previous item has been read)
      if (lane < 4) {
        G.lo[p] = lo; G.hi[p] = hi;
        G.first_tile[p] = p == 0 ? 0 : p == 1 ? t0 : p == 2 ? t0 + t1 : t0 + t1 + t2;
        G.krow[p] = p < 3 ? (int64_t)a0.x + d : (int64_t)h2.y + d;
        G.k2[p] = ptr_of(a1.x, a1.y) + (int64_t)d * kd.sub2;
        G.k4[p] = ptr_of(a1.z, a1.w) + (int64_t)d * kd.sub4;
        G.k8[p] = ptr_of(a2.x, a2.y) + (int64_t)d * kd.n8;
        G.vrow[p] = ptr_of(a2.z, a2.w) + (int64_t)d * phase_row_bytes(p);
        G.vrow_idx[p] = a0.z >= 0 ? a0.z + d : -1;
        if (p < 3) { G.sc[p] = ptr_of(a3.x, a3.y) + 2 * d; G.zp[p] = ptr_of(a3.z, a3.w) + 2 * d; }
      }
      if (lane == 0) G.vmaps = ptr_of(h2.z, h2.w);
      __syncwarp();
      const int total = fits ? t0 + t1 + t2 + t3 : 0;
      if (!fits && lane == 0 && status != nullptr) atomicOr(status, 2);
      const int n_it = max(total, 1);
      const uint64_t pol_stream = l2_policy_stream();
#if RDKV_STATIC_ROUNDS
      // the CTA's first rounds of items are dealt out statically (item = CTA + round * CTAs: the CTAs keep
      // pace while there is plenty of work), so the next item is known now and the lines of its unit
      // record and K slots can be on their way to L2 while this item's tiles are issued; only the last
      // round or two are drawn from the counter
      if (li + 1 < static_rounds) {
        const int ni = (int)blockIdx.x + (li + 1) * (int)gridDim.x;
        const int uy = ni < n_whole ? ni : n_whole + (ni - n_whole) / k_chunks;
        const int64_t nu = (int64_t)(uy / hy) * (H_q / g) + (uy % hy) / n_hgrp;
        if (lane < 3) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const unsigned char*>(unit_recs + nu) + 128 * lane));
        else if (lane - 3 < (nkb_max * 32 * (int)sizeof(KSlotRec) + 127) / 128)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const unsigned char*>(kslots + nu * nkb_max * 32) + 128 * (lane - 3)));
      }
#endif
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const int slot = it % PLAN_TILES;
        if (slot == 0) {                                   // plan tiles [it, it + 32)
          __syncwarp();
          if (it + lane < total) {
            const TileDesc t = tile_of<4>(G, it + lane);
            const int tp = t.phase;
            TilePlan& P = s_plan[lane];
            const unsigned char* a_k2 = G.k2[tp] + (int64_t)t.row0 * kd.sub2;
            const unsigned char* a_k4 = G.k4[tp] + (int64_t)t.row0 * kd.sub4;
            const unsigned char* a_k8 = G.k8[tp] + (int64_t)t.row0 * kd.n8;
            const unsigned char* a_v = G.vrow[tp] + (int64_t)t.row0 * phase_row_bytes(tp);
            const unsigned char* a_sc = G.sc[tp < 3 ? tp : 0] + t.row0 * 2;
            const unsigned char* a_zp = G.zp[tp < 3 ? tp : 0] + t.row0 * 2;
            // the V rows: one box of the phase's tensor map (src = the map, len = the box's bytes, dst_off = its
            // first row) when the table has maps, else copies by the lanes at the padded pitch
            // (a ragged last fp16 block goes that way too: the rows behind it are cleared)
            const bool v_tma = tp >= V_PAD_FROM && G.vmaps != nullptr && G.vrow_idx[tp] >= 0 && (tp < 3 || (t.n & 31) == 0);
            if (v_tma) P.rg[0] = RangePlan{G.vmaps + 128 * tp, phase_tile_rows(tp) * phase_pitch(tp), (uint32_t)(G.vrow_idx[tp] + t.row0)};
            else P.rg[0] = RangePlan{a_v, t.n * phase_row_bytes(tp), (uint32_t)SL.v};
            P.rg[1] = RangePlan{a_k2, t.n * kd.sub2, (uint32_t)SL.k2};
            P.rg[2] = RangePlan{a_k4, t.n * kd.sub4, (uint32_t)SL.k4};
            P.rg[3] = RangePlan{a_k8, t.n * kd.n8, (uint32_t)SL.k8};
            P.rg[4] = RangePlan{a_sc, tp < 3 ? t.n * 2 : 0, (uint32_t)SL.sc};
            P.rg[5] = RangePlan{a_zp, tp < 3 ? t.n * 2 : 0, (uint32_t)SL.zp};
            auto low4 = [](const unsigned char* x) { return (uint32_t)reinterpret_cast<uintptr_t>(x) & 15u; };
            int blocks_before = 0;
#pragma unroll
            for (int qq = 0; qq < 3; ++qq)
              if (qq < tp) blocks_before += (G.hi[qq] - G.lo[qq] + 31) >> 5;
            blocks_before += t.row0 >> 5;
            P.info.phase = tp | (blocks_before & (FW - 1)) << 8 | (v_tma ? 1 << 16 : tp >= V_PAD_FROM ? 1 << 17 : 0); P.info.n = t.n;
            P.info.offs = low4(a_k2) | low4(a_k4) << 4 | low4(a_k8) << 8 |
                          (tp < 3 ? low4(a_sc) << 16 | low4(a_zp) << 20 : 0u);
            P.info.krow0 = (int)(G.krow[tp] + t.row0);
          }
          __syncwarp();
        }
        const int gi = git + it, stage = gi % FSTAGES;
        const uint32_t sbu = smem0 + stage * stage_bytes;
        // lanes 0..5: the tile's six ranges; lanes 6, 7 with the item's first tile: its header
        RangePlan rp = {nullptr, 0, 0u};
        uint32_t dst = 0;
        TileInfo ti = {0, 0, 0u, 0};
        if (it < total) {
          ti = s_plan[slot].info;
          if (lane < 6) { rp = s_plan[slot].rg[lane]; dst = sbu + rp.dst_off; }
        }
        if (it == 0 && lane == 6) {
          rp.src = reinterpret_cast<const unsigned char*>(q) + ((int64_t)view_idx * H_q + hq0) * D * q_elt;
          rp.len = gcnt * D * q_elt; dst = smem_u32(hdr);
        }
        if (it == 0 && lane == 7) {
          rp.src = reinterpret_cast<const unsigned char*>(kslots + unit * nkb_max * 32);
          rp.len = nkb_max * 32 * (int)sizeof(KSlotRec); dst = smem_u32(hdr + hdr_q_bytes);
        }
        const bool v_tma = (ti.phase >> 16) & 1, v_lanes = (ti.phase >> 17) & 1;   // how the V rows travel
        const uintptr_t a = reinterpret_cast<uintptr_t>(rp.src), al = a & ~(uintptr_t)15;
        uint32_t bytes = rp.len > 0 ? (uint32_t)(((a + rp.len + 15) & ~(uintptr_t)15) - al) : 0u;
        if (lane == 0 && v_tma) bytes = (uint32_t)rp.len;  // (the whole box is counted, whatever part of it lies in the tensor)
        if (lane == 0 && v_lanes) bytes = 0u;
        uint32_t tx = bytes;
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
        if (gi >= FSTAGES) {                               // wait (bounded) until the compute warps have left the slot
          const uint32_t parity = ((gi / FSTAGES) - 1) & 1;
          unsigned spins = 0;
          while (!mbar_try_wait(&s_empty[stage], parity)) {
            if (++spins > WAIT_LIMIT) {
              if (lane == 0 && status != nullptr) atomicOr(status, 1);
              break;
            }
          }
        }
        if (lane == 0) mbar_expect_tx(&s_full[stage], tx);
        __syncwarp();
        {
          const bool by_map = lane == 0 && v_tma;
          tma_g2s_2d_if(by_map, sbu + SL.v, rp.src, 0, (int)rp.dst_off, &s_full[stage], pol_stream);
          bulk_g2s_hint_if(bytes != 0u && !by_map, dst, reinterpret_cast<const void*>(al), bytes, &s_full[stage], pol_stream);
        }
        if (v_lanes) {                                     // (here: a ragged last fp16 block; 16-byte aligned rows of 256 bytes)
          const unsigned char* vsrc = s_plan[slot].rg[0].src;
          const uint32_t vdst = sbu + SL.v;
#pragma unroll 1
          for (int b = lane; b < ti.n * 16; b += 32) cp16(vdst + (b >> 4) * phase_pitch(3) + 16 * (b & 15), vsrc + 16 * b);
        }
        if ((ti.phase & 3) == 3 && (ti.n & 31)) {          // fp16 phase: finite data past the tile's end
          const int first = ti.n * phase_pitch(3);
          const int last = min(((ti.n + 31) & ~31) * phase_pitch(3), V_STAGE);
          unsigned char* sv = smem_raw + (size_t)stage * stage_bytes + SL.v;
          for (int i = first + 4 * lane; i < last; i += 4 * 32) *reinterpret_cast<uint32_t*>(sv + i) = 0u;
        }
        if (lane == 0) {
          s_tile[stage] = ti;
          if (it == 0) s_item[li & 1] = ItemInfo{n2p, n4p, n8c, total, item, 0, 0, 0};
        }
        mbar_arrive_on_copies(&s_full[stage]);
        mbar_arrive(&s_full[stage]);
      }
      git += n_it;
      // the next item: drawn now, when this one's tiles are all on their way (the compute warps are
      // still two tiles behind), so that whichever CTA gets through its items first takes the next
#if RDKV_STATIC_ROUNDS
      if (li + 1 < static_rounds) next_item = (int)blockIdx.x + (li + 1) * (int)gridDim.x;   // (every lane; no round trip)
      else if (lane == 0) next_item = atomicAdd(work, 1) + static_rounds * (int)gridDim.x;
#else
      if (lane == 0) next_item = atomicAdd(work, 1) + (int)gridDim.x;
#endif
      item = __shfl_sync(0xffffffffu, next_item, 0);
    } else {
      // ── compute warps ──
      auto wait_tile = [&](int gi) {
        const int st = gi % FSTAGES;
        const uint32_t parity = (gi / FSTAGES) & 1;
        unsigned spins = 0;
        while (!mbar_try_wait(&s_full[st], parity)) {
          if (++spins > WAIT_LIMIT) {
            if (lane == 0 && status != nullptr) atomicOr(status, 1);
            break;
          }
        }
      };
      const ItemInfo ii = s_item[li & 1];                  // (the item's first tile, and with it its header, has landed)
      const int total_tiles = ii.total, n_it = max(total_tiles, 1);
      const KDims kd = k_dims(ii.n2p, ii.n4p, ii.n8c);
      const StageLayout SL = stage_layout(kd.sub2, kd.sub4, kd.n8);
      // fold the item's queries from its header: q*scale in MMA fragment order, zero-point bias
      {
        const KSlotRec* hk = reinterpret_cast<const KSlotRec*>(hdr + hdr_q_bytes);
        const bool head_ok = r < gcnt;
        const int qrow = (head_ok ? r : 0) * D;
        auto qload = [&](uint32_t ch) -> float {
          if (q_dtype == RDKV_F32) return reinterpret_cast<const float*>(hdr)[qrow + ch];
          const uint16_t x = reinterpret_cast<const uint16_t*>(hdr)[qrow + ch];
          return q_dtype == RDKV_BF16 ? __uint_as_float((uint32_t)x << 16) : h2f(x);
        };
        auto fold_block = [&](const KSlotRec& km, int kb, float& bias) {
          const int ex2b = kb < 2 * kd.nsp2 ? 4 * (kb & 1) : 0;
          const int exs = kb < 2 * kd.nsp2 ? 2 : kb < 2 * kd.nsp2 + 2 * kd.nsp4 ? 4 : 0;
          float val[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ex = ex2b + (e >> 1) * exs;
            const float scv = h2f((uint16_t)((e < 2 ? km.sc01 : km.sc23) >> (16 * (e & 1))));
            const float zpv = (float)((km.zp4 >> (8 * e)) & 255u);
            float x = __half2float(__float2half_rn(qload((km.perm4 >> (8 * e)) & 127u) * scv * pow2i(-ex)));
            if (!head_ok) x = 0.f;
            bias += zpv * (x * pow2i(ex));
            val[e] = x;
          }
          qsA[kb * 32 + lane] = make_uint2(pack_h2(val[0], val[1]), pack_h2(val[2], val[3]));
        };
        // one copy of the fold code (it runs once per item, from a cold instruction cache); the sums
        // are formed as in the one-item form of the kernel: the first two blocks of a warp on their own
        // and then added, further blocks term by term
        float bias_part = 0.f;
        int nb = 0;
#pragma unroll 1
        for (int kb = warp; kb < kd.nkb; kb += FW, ++nb) {
          float b = nb < 2 ? 0.f : bias_part;
          fold_block(hk[kb * 32 + lane], kb, b);
          bias_part = nb < 2 ? bias_part + b : b;
        }
        bias_part += __shfl_xor_sync(0xffffffffu, bias_part, 1);
        bias_part += __shfl_xor_sync(0xffffffffu, bias_part, 2);
        if (j == 0) s_bias[warp][r] = bias_part;
        bar_sync(BAR_COMPUTE, FW * 32);
      }
      // (written after the barrier: every warp has left the previous item's merge, which reads it)
      {
        const int n_chunks_ = n_chunks;
        float* rec_base = (n_chunks_ > 1 || merged == nullptr) ? partials : merged;
        if (tid == 0) {
          s_epi.out_rows = out != nullptr ? out + ((int64_t)view_idx * H_q + hq0) * D : nullptr;
          s_epi.rec0 = rec_base != nullptr
                           ? rec_base + ((int64_t)(view_idx * H_q + hq0) * n_chunks_ + chunk) * RDKV_PARTIAL_STRIDE
                           : nullptr;
          s_epi.rec_stride = (int64_t)n_chunks_ * RDKV_PARTIAL_STRIDE;
          s_epi.row0 = (int64_t)view_idx * H_q + hq0;
          s_epi.how = (n_chunks_ == 1 && out != nullptr) ? 1 : 0;
          s_epi.gcnt = gcnt; s_epi.n_chunks = n_chunks_; s_epi.unit_y = unit_y;
        }
      }
  constexpr bool TAIL = false, ATTN = MODE == MODE_ATTN;   // (no uncompressed tail in this form)
  float tref_e = 0.f, tref_o = 0.f;
  const uint32_t qt_lane = 0u;
  const bool tail_bf = false;
#include "decode_state.inc"
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const int stage = (git + it) % FSTAGES;
        if (it > 0) wait_tile(git + it);
        const TileInfo t = s_tile[stage];
        const int p = t.phase & 3;
        const int nblocks = (t.n + 31) >> 5;
        const int pb = (warp + FW - (it * (TILE_MAX / 128)) % FW) % FW;
#include "decode_tile.inc"
        if (it + 1 < n_it) {                               // (the item's last slot is handed back after the merge)
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_empty[stage]);
        }
      }
      const int last_stage = (git + n_it - 1) % FSTAGES;
      // ── merge the four workers and write the item's result (in the ring slot of its last tile) ──
      if (cur_phase >= 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float f = pow2i(acc_exp(cur_phase, i & 3));
          acc[i][0] *= f; acc[i][1] *= f; acc[i][2] *= f; acc[i][3] *= f;
        }
      }
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l_e += __shfl_xor_sync(0xffffffffu, l_e, o); l_o += __shfl_xor_sync(0xffffffffu, l_o, o);
      }
      bar_sync(BAR_COMPUTE, FW * 32);                      // every worker is done with its stages
      float* red = reinterpret_cast<float*>(smem_raw + (size_t)last_stage * stage_bytes);   // [FW][GH][128]
      if (r == 0) {
        s_ml[warp][2 * j][0] = m_e; s_ml[warp][2 * j][1] = l_e; s_ml[warp][2 * j][2] = zacc[0];
        s_ml[warp][2 * j + 1][0] = m_o; s_ml[warp][2 * j + 1][1] = l_o; s_ml[warp][2 * j + 1][2] = zacc[1];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int ch = 4 * r + 2 * (i >> 2) + 32 * (i & 3);
        float* o0 = red + ((warp * GH + 2 * j) * D);
        float* o1 = o0 + D;
        o0[ch] = acc[i][0]; o1[ch] = acc[i][1]; o0[ch + 1] = acc[i][2]; o1[ch + 1] = acc[i][3];
      }
      bar_sync(BAR_COMPUTE, FW * 32);
      const EpiInfo ep = s_epi;
      final_merge<true>(red, &s_ml[0][0][0], ep.gcnt, ep.how, ep.out_rows, ep.rec0, ep.rec_stride);
      if (ep.n_chunks > 1 && unit_ctr != nullptr)
        chunk_merge<true>(partials, unit_ctr + ep.unit_y, ep.n_chunks, ep.gcnt, ep.row0, out, merged);
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[last_stage]);    // only now may the staging warp refill the slot
      git += n_it;
    }
  }
  if (warp == FW) cp_wait<0>();
}

}  // namespace rdkv

using namespace rdkv;

extern "C" int rdkv_decode_stage_bytes(int k_row_bytes_max) { return align128i(stage_capacity(k_row_bytes_max)); }

// Prepared table of a set of views: per (view, KV head) a UnitRec (row counts, whole-head
// alignment flag) and the K slot quadruples in the order the fused kernel's threads consume them.
// With it a CTA needs ONE round trip to global memory (view record, unit record, slots and query
// rows together) before its staging warp can plan copies and its compute warps can fold the
// queries; without it the counts, scales, zero points and permutation cost a second, dependent
// round trip and the slot arithmetic is redone by every CTA.  One block per unit.
__global__ void __launch_bounds__(128)
decode_prepare_kernel(const rdkv_layer_view* __restrict__ views, int H_kv, int nkb_max,
                      UnitRec* __restrict__ recs, KSlotRec* __restrict__ kslots, const unsigned char* __restrict__ v_maps) {
  const int64_t unit = blockIdx.x;
  const rdkv_layer_view& v = views[unit / H_kv];
  const int h = (int)(unit % H_kv);
  const KDims kd = k_dims(v.n_ch2_pad, v.n_ch4_pad, v.n_ch8);
  const int d_pad = kd.n2p + kd.n4p + kd.n8;
  const uint16_t* sc = v.k_scale + (int64_t)h * d_pad;
  const uint16_t* zp = v.k_zp + (int64_t)h * d_pad;
  const int64_t* perm = v.k_perm + (int64_t)h * v.k_perm_head_stride;
  for (int i = threadIdx.x; i < nkb_max * 32; i += blockDim.x) {
    const int kb = i >> 5, j = i & 3;
    KSlotRec rec = {0u, 0u, 0u, 0u};
    if (kb < kd.nkb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float f;
        const int slot = k_slot(kd, kb, j, e, &f);
        if (slot < 0) continue;
        const uint32_t pm = (uint32_t)(perm[slot] & (D - 1));
        const uint32_t z = (uint32_t)min(255.f, fmaxf(0.f, h2f(zp[slot])));
        rec.perm4 |= pm << (8 * e);
        rec.zp4 |= z << (8 * e);
        if (e < 2) rec.sc01 |= (uint32_t)sc[slot] << (16 * e); else rec.sc23 |= (uint32_t)sc[slot] << (16 * (e - 2));
      }
    }
    kslots[unit * nkb_max * 32 + i] = rec;
  }
  if (threadIdx.x == 0) {
    const HeadCounts hc = head_counts(v, h);
    bool fast = true, mapped = true;                      // mapped: the V rows of every spaced-out phase can come through a tensor map
    UnitRec u;
    for (int p = 0; p < 4; ++p) {                          // the whole head, phase by phase (as the kernel's geometry does per chunk)
      const int lo = p == 0 ? 0 : p == 1 ? hc.n2 : p == 2 ? hc.n2 + hc.n4 : hc.t_v;
      const int hi = p == 0 ? hc.n2 : p == 1 ? hc.n2 + hc.n4 : p == 2 ? hc.t_v : hc.t_v + hc.n16;
      const int n = hi - lo;
      const int64_t krow = p < 3 ? lo : (int64_t)v.max_t_v;
      const unsigned char* a2 = kd.sub2 ? v.k2 + h * v.k2_head_stride + krow * kd.sub2 : nullptr;
      const unsigned char* a4 = kd.sub4 ? v.k4 + h * v.k4_head_stride + krow * kd.sub4 : nullptr;
      const unsigned char* a8 = kd.n8 ? v.k8 + h * v.k8_head_stride + krow * kd.n8 : nullptr;
      const unsigned char* vlo = p == 0 ? v.v2 : p == 1 ? v.v4 : p == 2 ? v.v8 : reinterpret_cast<const unsigned char*>(v.v16);
      const int64_t vext = p == 0 ? v.v2_bytes : p == 1 ? v.v4_bytes : p == 2 ? v.v8_bytes : v.v16_bytes;
      const int64_t vhs = p == 0 ? v.v2_head_stride : p == 1 ? v.v4_head_stride : p == 2 ? v.v8_head_stride : 2 * v.v16_head_stride;
      const unsigned char* vb = vlo != nullptr ? vlo + h * vhs : nullptr;
      const unsigned char* scb = reinterpret_cast<const unsigned char*>(v.v_scale);
      const unsigned char* zpb = reinterpret_cast<const unsigned char*>(v.v_zp);
      const unsigned char* gsc = p < 3 && scb != nullptr ? scb + (h * v.v_meta_head_stride + lo) * 2 : nullptr;
      const unsigned char* gzp = p < 3 && zpb != nullptr ? zpb + (h * v.v_meta_head_stride + lo) * 2 : nullptr;
      if (n > 0) {
        if (kd.sub2) fast = fast && blocks_inside(a2, a2 + (int64_t)n * kd.sub2, v.k2, v.k2 + v.k2_bytes);
        if (kd.sub4) fast = fast && blocks_inside(a4, a4 + (int64_t)n * kd.sub4, v.k4, v.k4 + v.k4_bytes);
        if (kd.n8) fast = fast && blocks_inside(a8, a8 + (int64_t)n * kd.n8, v.k8, v.k8 + v.k8_bytes);
        fast = fast && vb != nullptr && blocks_inside(vb, vb + (int64_t)n * phase_row_bytes(p), vlo, vlo + vext);
        if (p < 3) {
          fast = fast && gsc != nullptr && gzp != nullptr;
          fast = fast && blocks_inside(gsc, gsc + n * 2, scb, scb + v.v_meta_bytes);
          fast = fast && blocks_inside(gzp, gzp + n * 2, zpb, zpb + v.v_meta_bytes);
        }
      }
      // row lo's number in the phase's tensor map (a map whose first 16 bytes are zero was not encoded)
      int v_row = -1;
      if (v_maps != nullptr && vb != nullptr && n > 0) {
        const int4 m0 = *reinterpret_cast<const int4*>(v_maps + ((unit / H_kv) * 4 + p) * 128);
        const int64_t delta = vb - vlo;
        const int rb = phase_row_bytes(p);
        if ((m0.x | m0.y | m0.z | m0.w) != 0 && delta >= 0 && delta % rb == 0 && delta / rb + n < 0x7fffffffLL) v_row = (int)(delta / rb);
      }
      if (n > 0 && p >= V_PAD_FROM && v_row < 0) mapped = false;
      u.ph[p].b_lo = lo; u.ph[p].b_hi = hi; u.ph[p].v_row = v_row; u.ph[p].pad1 = 0;
      u.ph[p].k2 = a2; u.ph[p].k4 = a4; u.ph[p].k8 = a8; u.ph[p].vrow = vb; u.ph[p].sc = gsc; u.ph[p].zp = gzp;
    }
    u.n2 = hc.n2; u.n4 = hc.n4; u.n8 = hc.n8; u.n16 = hc.n16;
    u.flags = (fast ? 1 : 0) | (fast && mapped ? 2 : 0); u.nkb = kd.nkb; u.n_ch2_pad = kd.n2p; u.n_ch4_pad = kd.n4p;
    u.n_ch8 = kd.n8; u.max_t_v = v.max_t_v;
    const uintptr_t vm = v_maps != nullptr ? reinterpret_cast<uintptr_t>(v_maps + (unit / H_kv) * 4 * 128) : 0;
    u.vmaps_lo = (unsigned)(vm & 0xFFFFFFFFu); u.vmaps_hi = (unsigned)(vm >> 32);
    recs[unit] = u;
  }
}

template <int MODE>
static int launch_fused(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q, int H_kv,
                        int chunk_rows, int n_chunks, int k_row_bytes_max, float* partials, float* out, int* status,
                        float* aux, int64_t aux_stride, int t_eff, void* stream,
                        const void* unit_recs = nullptr, const void* kslots = nullptr, int nkb_max = 0,
                        int* unit_ctr = nullptr, float* merged = nullptr,
                        int row_begin = 0, int row_end = 0x7fffffff, int n_whole = 0, int part = 0, int parts = 1,
                        const TailArgs* tail = nullptr) {
  const int g = H_q / H_kv;
  const int n_hgrp = (g + GH - 1) / GH;
  const int64_t units = (int64_t)n_views * H_kv * n_hgrp;
  if (n_whole < 0 || n_whole > units) return RDKV_ERR_BAD_ARG;
  const int64_t items = n_whole + (units - n_whole) * n_chunks;
  if (items > 0x7fffffffLL) return RDKV_ERR_TOO_LARGE;
  // results and records are written four floats at a time
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(partials) & 15) ||
      (reinterpret_cast<uintptr_t>(merged) & 15))
    return RDKV_ERR_BAD_ARG;
  const int stage_bytes = align128i(stage_capacity(k_row_bytes_max));   // (a tile's V box lands on a 128-byte boundary)
  const int qs_bytes = (nkb_max > 0 ? std::min(nkb_max, KB_MAX) : KB_MAX) * 256;   // (as the kernel lays it out)
  size_t smem = (size_t)FSTAGES * stage_bytes + qs_bytes + FOLD_Q_BYTES + FOLD_META_BYTES +
                (MODE == MODE_ATTN_TAIL ? TAIL_EXTRA_BYTES : 0);
  const size_t epilogue = (size_t)FW * GH * D * sizeof(float);
  if (smem < epilogue) smem = epilogue;
  if (smem > 227 * 1024) return RDKV_ERR_TOO_LARGE;
  TailArgs ta;
  memset(&ta, 0, sizeof(ta));
  if (tail != nullptr) ta = *tail;
  cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  decode_fused_kernel<MODE><<<(unsigned)items, CTA_THREADS, smem, (cudaStream_t)stream>>>(
      views, q, q_dtype, H_q, g, chunk_rows, n_chunks, n_whole, stage_bytes, partials, out, status, aux, aux_stride, t_eff,
      reinterpret_cast<const UnitRec*>(unit_recs), reinterpret_cast<const KSlotRec*>(kslots), nkb_max, unit_ctr, merged,
      row_begin, row_end, part, parts, ta);
  return launch_status();
}

static int check_fused_args(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q, int H_kv,
                            int k_row_bytes_max) {
  if (views == nullptr || q == nullptr || n_views < 0) return RDKV_ERR_BAD_ARG;
  if (q_dtype < RDKV_F16 || q_dtype > RDKV_F32) return RDKV_ERR_BAD_ARG;
  if (H_q <= 0 || H_kv <= 0 || H_q % H_kv != 0) return RDKV_ERR_BAD_SHAPE;
  if (k_row_bytes_max <= 0 || k_row_bytes_max > 224) return RDKV_ERR_BAD_SHAPE;
  return RDKV_OK;
}

extern "C" int rdkv_decode_attn_partial(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype,
                                        int H_q, int H_kv, int chunk_rows, int n_chunks, int k_row_bytes_max,
                                        float* partials, float* out, int* status, void* stream) {
  if (n_chunks <= 0 || chunk_rows <= 0) return RDKV_ERR_BAD_ARG;
  if (partials == nullptr && !(n_chunks == 1 && out != nullptr)) return RDKV_ERR_BAD_ARG;
  const int rc = check_fused_args(views, n_views, q, q_dtype, H_q, H_kv, k_row_bytes_max);
  if (rc != RDKV_OK || n_views == 0) return rc;
  return launch_fused<MODE_ATTN>(views, n_views, q, q_dtype, H_q, H_kv, chunk_rows, n_chunks, k_row_bytes_max,
                                 partials, out, status, nullptr, 0, 0, stream);
}

extern "C" int rdkv_decode_k_blocks(int n_ch2_pad, int n_ch4_pad, int n_ch8) {
  return k_dims(n_ch2_pad, n_ch4_pad, n_ch8).nkb;
}

extern "C" int64_t rdkv_decode_prepared_bytes(int64_t n_units, int nkb_max, int which) {
  if (n_units < 0 || nkb_max < 0) return -1;
  return which == 0 ? n_units * (int64_t)sizeof(UnitRec) : n_units * nkb_max * 32 * (int64_t)sizeof(KSlotRec);
}

// The driver's tensor-map encoder, found through the runtime (the library does not link the driver).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn v_map_encoder() {
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

extern "C" int64_t rdkv_decode_v_map_bytes(int n_views) { return n_views < 0 ? -1 : (int64_t)n_views * 4 * (int64_t)sizeof(CUtensorMap); }

extern "C" int rdkv_decode_encode_v_maps(const rdkv_layer_view* views_host, int n_views, void* maps_host) {
  static_assert(sizeof(CUtensorMap) == 128, "a tensor map is 128 bytes");
  if (views_host == nullptr || maps_host == nullptr || n_views < 0) return -1;
  memset(maps_host, 0, (size_t)n_views * 4 * sizeof(CUtensorMap));
  EncodeTiledFn enc = v_map_encoder();
  if (enc == nullptr) return 0;
  int done = 0;
  for (int i = 0; i < n_views; ++i) {
    const rdkv_layer_view& v = views_host[i];
    for (int p = 0; p < 4; ++p) {
      const void* base = p == 0 ? (const void*)v.v2 : p == 1 ? (const void*)v.v4 : p == 2 ? (const void*)v.v8 : (const void*)v.v16;
      const int64_t bytes = p == 0 ? v.v2_bytes : p == 1 ? v.v4_bytes : p == 2 ? v.v8_bytes : v.v16_bytes;
      const int rb = phase_row_bytes(p);
      if (base == nullptr || bytes < rb || (reinterpret_cast<uintptr_t>(base) & 15) != 0) continue;
      const int64_t rows = bytes / rb;
      if (rows > 0x7fffffffLL) continue;
      // the tensor as rows of rb bytes (fp16 rows as 128 16-bit elements: a box is at most 256 elements wide);
      // the box is one tile of rows, V_PAD bytes wider than a row: the excess arrives as zeros and
      // spaces the rows in shared memory
      CUtensorMap* tm = reinterpret_cast<CUtensorMap*>(maps_host) + (size_t)i * 4 + p;
      const int es = p == 3 ? 2 : 1;
      const cuuint64_t dims[2] = {(cuuint64_t)(rb / es), (cuuint64_t)rows};
      const cuuint64_t strides[1] = {(cuuint64_t)rb};
      const cuuint32_t box[2] = {(cuuint32_t)(phase_pitch(p) / es), (cuuint32_t)phase_tile_rows(p)};
      const cuuint32_t elem[2] = {1u, 1u};
      const CUresult r = enc(tm, p == 3 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base),
                             dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) memset(tm, 0, sizeof(CUtensorMap));
      else ++done;
    }
  }
  return done;
}

extern "C" int rdkv_decode_prepare(const rdkv_layer_view* views, int n_views, int H_kv, int nkb_max, void* unit_recs,
                                   void* k_slots, const void* v_maps, void* stream) {
  if (views == nullptr || unit_recs == nullptr || k_slots == nullptr || n_views < 0 || H_kv <= 0) return RDKV_ERR_BAD_ARG;
  if (nkb_max <= 0 || nkb_max > KB_MAX) return RDKV_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(unit_recs) & 15) || (reinterpret_cast<uintptr_t>(k_slots) & 15)) return RDKV_ERR_BAD_ARG;
  const int64_t n = (int64_t)n_views * H_kv;
  if (n == 0) return RDKV_OK;
  if (n > 0x7fffffffLL) return RDKV_ERR_TOO_LARGE;
  if (reinterpret_cast<uintptr_t>(v_maps) & 63) return RDKV_ERR_BAD_ARG;
  decode_prepare_kernel<<<(unsigned)n, 128, 0, (cudaStream_t)stream>>>(
      views, H_kv, nkb_max, reinterpret_cast<UnitRec*>(unit_recs), reinterpret_cast<KSlotRec*>(k_slots),
      reinterpret_cast<const unsigned char*>(v_maps));
  return launch_status();
}

extern "C" int rdkv_decode_attn(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q,
                                int H_kv, int chunk_rows, int n_chunks, int n_whole_units, int row_begin, int row_end,
                                int seq_part, int seq_parts, int k_row_bytes_max, const void* unit_recs, const void* k_slots, int nkb_max,
                                float* partials, int32_t* unit_counters, float* out, float* out_record,
                                int32_t* status, void* stream) {
  if (n_chunks <= 0 || chunk_rows <= 0 || row_begin < 0 || row_end < row_begin) return RDKV_ERR_BAD_ARG;
  if (seq_parts < 1 || seq_part < 0 || seq_part >= seq_parts) return RDKV_ERR_BAD_ARG;
  if ((out == nullptr) == (out_record == nullptr)) return RDKV_ERR_BAD_ARG;          // exactly one result form
  if (n_chunks > 1 && (partials == nullptr || unit_counters == nullptr)) return RDKV_ERR_BAD_ARG;
  if ((unit_recs == nullptr) != (k_slots == nullptr)) return RDKV_ERR_BAD_ARG;
  if (unit_recs != nullptr && ((reinterpret_cast<uintptr_t>(unit_recs) & 15) || (reinterpret_cast<uintptr_t>(k_slots) & 15) ||
                               nkb_max <= 0 || nkb_max > KB_MAX))
    return RDKV_ERR_BAD_ARG;
  const int rc = check_fused_args(views, n_views, q, q_dtype, H_q, H_kv, k_row_bytes_max);
  if (rc != RDKV_OK || n_views == 0) return rc;
  return launch_fused<MODE_ATTN>(views, n_views, q, q_dtype, H_q, H_kv, chunk_rows, n_chunks, k_row_bytes_max,
                                 partials, out, status, nullptr, 0, 0, stream, unit_recs, k_slots, nkb_max,
                                 unit_counters, out_record, row_begin, row_end, n_whole_units, seq_part, seq_parts);
}

extern "C" int rdkv_decode_attn_tail(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q,
                                     int H_kv, int chunk_rows, int n_chunks, int n_whole_units, int row_begin,
                                     int row_end, int seq_part, int seq_parts, int k_row_bytes_max,
                                     const void* unit_recs, const void* k_slots, int nkb_max, float* partials,
                                     int32_t* unit_counters, float* out, float* out_record, int32_t* status,
                                     const rdkv_tail_args* tail, void* stream) {
  if (tail == nullptr) return RDKV_ERR_BAD_ARG;
  if (n_chunks <= 0 || chunk_rows <= 0 || row_begin < 0 || row_end < row_begin) return RDKV_ERR_BAD_ARG;
  if (seq_parts < 1 || seq_part < 0 || seq_part >= seq_parts) return RDKV_ERR_BAD_ARG;
  if ((out == nullptr) == (out_record == nullptr)) return RDKV_ERR_BAD_ARG;
  if (n_chunks > 1 && (partials == nullptr || unit_counters == nullptr)) return RDKV_ERR_BAD_ARG;
  if ((unit_recs == nullptr) != (k_slots == nullptr)) return RDKV_ERR_BAD_ARG;
  if (unit_recs != nullptr && ((reinterpret_cast<uintptr_t>(unit_recs) & 15) || (reinterpret_cast<uintptr_t>(k_slots) & 15) ||
                               nkb_max <= 0 || nkb_max > KB_MAX))
    return RDKV_ERR_BAD_ARG;
  const rdkv_tail_args& t = *tail;
  if (t.dtype != RDKV_F16 && t.dtype != RDKV_BF16) return RDKV_ERR_BAD_ARG;
  if (t.cap < 0 || t.n_new < 0 || t.n_new > t.cap) return RDKV_ERR_BAD_ARG;
  const bool rows = t.cap > 0 && (t.n_new > 0 || t.n_new_per_view != nullptr || t.append);
  if (rows) {                                              // the staged rows: 16-byte aligned whatever the view, head and row
    if (t.new_k == nullptr || t.new_v == nullptr) return RDKV_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(t.new_k) & 15) || (reinterpret_cast<uintptr_t>(t.new_v) & 15) ||
        (t.view_stride & 7) || (t.head_stride & 7))
      return RDKV_ERR_BAD_SHAPE;
  }
  if ((t.rope_cos == nullptr) != (t.rope_sin == nullptr)) return RDKV_ERR_BAD_ARG;
  if (t.rope_cos != nullptr && (t.rope_dtype < RDKV_F16 || t.rope_dtype > RDKV_F32)) return RDKV_ERR_BAD_ARG;
  if ((t.k_cur == nullptr) != (t.v_cur == nullptr)) return RDKV_ERR_BAD_ARG;
  if (t.append && (t.k_cur == nullptr || t.new_k == nullptr || t.new_v == nullptr)) return RDKV_ERR_BAD_ARG;
  if (t.append && t.n_new_per_view == nullptr && t.n_new >= t.cap) return RDKV_ERR_TOO_LARGE;
  const int rc = check_fused_args(views, n_views, q, q_dtype, H_q, H_kv, k_row_bytes_max);
  if (rc != RDKV_OK || n_views == 0) return rc;
  return launch_fused<MODE_ATTN_TAIL>(views, n_views, q, q_dtype, H_q, H_kv, chunk_rows, n_chunks, k_row_bytes_max,
                                      partials, out, status, nullptr, 0, 0, stream, unit_recs, k_slots, nkb_max,
                                      unit_counters, out_record, row_begin, row_end, n_whole_units, seq_part,
                                      seq_parts, tail);
}

// fused_rope on its own (rows of q and k rotated in place): one warp per row, lane i takes the
// channel pairs (i, i + 64) and (i + 32, i + 96).
namespace rdkv {
__global__ void __launch_bounds__(128)
rope_kernel(void* q, int q_dtype, int n_q, int64_t q_row_stride, void* k, int k_dtype, int n_k, int64_t k_row_stride,
            const void* cos_half, const void* sin_half, int cs_dtype) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_q + n_k) return;
  const bool is_q = row < n_q;
  void* base = is_q ? q : k;
  const int dt = is_q ? q_dtype : k_dtype;
  const int64_t off = is_q ? (int64_t)row * q_row_stride : (int64_t)(row - n_q) * k_row_stride;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = lane + 32 * u;
    const float c = load_q(cos_half, cs_dtype, i), sn = load_q(sin_half, cs_dtype, i);
    const float lo = load_q(base, dt, off + i), hi = load_q(base, dt, off + i + 64);
    const float a = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn)), b = __fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, sn));
    if (dt == RDKV_F16) {
      reinterpret_cast<__half*>(base)[off + i] = __float2half_rn(a);
      reinterpret_cast<__half*>(base)[off + i + 64] = __float2half_rn(b);
    } else if (dt == RDKV_BF16) {
      reinterpret_cast<__nv_bfloat16*>(base)[off + i] = __float2bfloat16_rn(a);
      reinterpret_cast<__nv_bfloat16*>(base)[off + i + 64] = __float2bfloat16_rn(b);
    } else {
      reinterpret_cast<float*>(base)[off + i] = a;
      reinterpret_cast<float*>(base)[off + i + 64] = b;
    }
  }
}
}  // namespace rdkv

extern "C" int rdkv_rope(void* q, int q_dtype, int n_q, int64_t q_row_stride, void* k, int k_dtype, int n_k,
                         int64_t k_row_stride, const void* cos_half, const void* sin_half, int cs_dtype,
                         void* stream) {
  if (n_q < 0 || n_k < 0 || cos_half == nullptr || sin_half == nullptr) return RDKV_ERR_BAD_ARG;
  if ((n_q > 0 && q == nullptr) || (n_k > 0 && k == nullptr)) return RDKV_ERR_BAD_ARG;
  for (int dt : {n_q > 0 ? q_dtype : RDKV_F16, n_k > 0 ? k_dtype : RDKV_F16, cs_dtype})
    if (dt < RDKV_F16 || dt > RDKV_F32) return RDKV_ERR_BAD_ARG;
  const int n = n_q + n_k;
  if (n == 0) return RDKV_OK;
  rope_kernel<<<(n + 3) / 4, 128, 0, (cudaStream_t)stream>>>(q, q_dtype, n_q, q_row_stride, k, k_dtype, n_k, k_row_stride,
                                                           cos_half, sin_half, cs_dtype);
  return launch_status();
}

extern "C" int rdkv_decode_attn_persistent(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype,
                                           int H_q, int H_kv, int chunk_rows, int n_chunks, int n_whole_units,
                                           int row_begin, int row_end, int seq_part, int seq_parts,
                                           int k_row_bytes_max, const void* unit_recs, const void* k_slots,
                                           int nkb_max, float* partials, int32_t* unit_counters,
                                           int32_t* work_counters, float* out, float* out_record, int32_t* status,
                                           void* stream) {
  if (work_counters == nullptr) return RDKV_ERR_BAD_ARG;
  if (n_chunks <= 0 || chunk_rows <= 0 || row_begin < 0 || row_end < row_begin) return RDKV_ERR_BAD_ARG;
  if (seq_parts < 1 || seq_part < 0 || seq_part >= seq_parts) return RDKV_ERR_BAD_ARG;
  if ((out == nullptr) == (out_record == nullptr)) return RDKV_ERR_BAD_ARG;
  if (n_chunks > 1 && (partials == nullptr || unit_counters == nullptr)) return RDKV_ERR_BAD_ARG;
  if (unit_recs == nullptr || k_slots == nullptr || nkb_max <= 0 || nkb_max > KB_MAX) return RDKV_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(unit_recs) & 15) || (reinterpret_cast<uintptr_t>(k_slots) & 15) ||
      (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(partials) & 15) || (reinterpret_cast<uintptr_t>(out_record) & 15))
    return RDKV_ERR_BAD_ARG;
  const int rc = check_fused_args(views, n_views, q, q_dtype, H_q, H_kv, k_row_bytes_max);
  if (rc != RDKV_OK || n_views == 0) return rc;
  const int g = H_q / H_kv;
  const int n_hgrp = (g + GH - 1) / GH;
  const int64_t units = (int64_t)n_views * H_kv * n_hgrp;
  if (n_whole_units < 0 || n_whole_units > units) return RDKV_ERR_BAD_ARG;
  const int64_t items = n_whole_units + (units - n_whole_units) * n_chunks;
  if (items > 0x7fffffffLL) return RDKV_ERR_TOO_LARGE;
  const int stage_bytes = align128i(stage_capacity(k_row_bytes_max));   // (a tile's V box lands on a 128-byte boundary)
  const int q_elt = q_dtype == RDKV_F32 ? 4 : 2;
  size_t smem = (size_t)FSTAGES * stage_bytes + (size_t)nkb_max * 256 +
                2 * ((size_t)GH * D * q_elt + (size_t)nkb_max * 32 * sizeof(KSlotRec));
  const size_t epilogue = (size_t)FW * GH * D * sizeof(float);
  if ((size_t)stage_bytes < epilogue) return RDKV_ERR_BAD_SHAPE;     // the merge works inside one ring slot
  if (smem > 227 * 1024) return RDKV_ERR_TOO_LARGE;
  cudaError_t e = cudaFuncSetAttribute(decode_persist_kernel<MODE_ATTN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return RDKV_ERR_LAUNCH; }
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_persist_kernel<MODE_ATTN>, CTA_THREADS, smem) != cudaSuccess ||
      per_sm <= 0) {
    g_last_cuda_error = (int)cudaGetLastError();
    return RDKV_ERR_LAUNCH;
  }
  const int64_t slots = (int64_t)sms * per_sm;
  const unsigned grid = (unsigned)(items < slots ? items : slots);
  decode_persist_kernel<MODE_ATTN><<<grid, CTA_THREADS, smem, (cudaStream_t)stream>>>(
      q, q_dtype, H_q, g, chunk_rows, n_chunks, n_whole_units, (int)items, stage_bytes, partials, out, status,
      reinterpret_cast<const UnitRec*>(unit_recs), reinterpret_cast<const KSlotRec*>(k_slots), nkb_max, unit_counters,
      out_record, row_begin, row_end, seq_part, seq_parts, work_counters);
  return launch_status();
}

extern "C" int rdkv_decode_scores(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q,
                                  int H_kv, int chunk_rows, int n_chunks, int k_row_bytes_max, int t_eff,
                                  float* scores, int64_t scores_row_stride, int* status, void* stream) {
  if (n_chunks <= 0 || chunk_rows <= 0 || scores == nullptr || t_eff < 0 || scores_row_stride < t_eff)
    return RDKV_ERR_BAD_ARG;
  if (n_views > 1) return RDKV_ERR_BAD_ARG;                 // one score matrix per call
  const int rc = check_fused_args(views, n_views, q, q_dtype, H_q, H_kv, k_row_bytes_max);
  if (rc != RDKV_OK || n_views == 0 || t_eff == 0) return rc;
  return launch_fused<MODE_SCORES>(views, n_views, q, q_dtype, H_q, H_kv, chunk_rows, n_chunks, k_row_bytes_max,
                                   nullptr, nullptr, status, scores, scores_row_stride, t_eff, stream);
}

extern "C" int rdkv_decode_weighted_sum(const rdkv_layer_view* views, int n_views, int H_q, int H_kv, int unit_rows,
                                        int k_row_bytes_max, const float* weights, int64_t weights_row_stride,
                                        float* out, int* status, void* stream) {
  if (unit_rows <= 0 || weights == nullptr || out == nullptr || weights_row_stride < 0) return RDKV_ERR_BAD_ARG;
  if (n_views > 1) return RDKV_ERR_BAD_ARG;                 // one weight matrix per call
  const int rc = check_fused_args(views, n_views, weights, RDKV_F32, H_q, H_kv, k_row_bytes_max);
  if (rc != RDKV_OK || n_views == 0) return rc;
  return launch_fused<MODE_WEIGHTS>(views, n_views, weights, RDKV_F32, H_q, H_kv, unit_rows, 1, k_row_bytes_max,
                                    nullptr, out, status, const_cast<float*>(weights), weights_row_stride, 0, stream);
}
