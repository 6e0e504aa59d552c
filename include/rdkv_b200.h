/*
 * rdkv_b200 — C ABI of the B200 (sm_100a) packed-KV decode path.
 *
 * Every entry point takes raw device pointers, explicit extents/strides and a
 * cudaStream_t (passed as void*), returns an int status (0 = RDKV_OK) and never
 * throws, aborts, allocates or synchronises unless its comment says otherwise.
 * Kernels are enqueued on the given stream only, so calls may be recorded into
 * a CUDA graph on a capturing stream.
 *
 * Each declaration names the reference interface it replaces, as
 * file:line inside the reference project (Junkai1860/RDKV).
 */
#ifndef RDKV_B200_H
#define RDKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ── status codes ─────────────────────────────────────────────────────────── */
enum {
  RDKV_OK = 0,
  RDKV_ERR_BAD_ARG = 1,      /* null pointer, negative extent, unsupported dtype      */
  RDKV_ERR_BAD_SHAPE = 2,    /* head_dim != 128, H_q % H_kv != 0, group size > 16 ... */
  RDKV_ERR_TOO_LARGE = 3,    /* extent beyond what the kernel (or its scratch) holds  */
  RDKV_ERR_LAUNCH = 4,       /* the CUDA runtime refused the launch (see cuda code)   */
  RDKV_ERR_NO_DEVICE = 5
};

/* element type tags for query tensors */
enum { RDKV_F16 = 0, RDKV_BF16 = 1, RDKV_F32 = 2 };

#define RDKV_HEAD_DIM 128
/* floats per split-sequence partial record: [0]=m (running max, log domain),
 * [1]=l (sum of exp), [2..3]=0, [4..131]=o (un-normalised output, 128 channels) */
#define RDKV_PARTIAL_STRIDE 132

/*
 * One (sequence, layer) of packed cache: H_kv heads in the reference's stacked
 * per-head layout (PackedKVLayer, obkv_accel/packing.py:43-111, plus the fp16
 * "Zone B" values TriZoneCache.new_v_only, packing.py:114-135).
 *
 * K token axis ("stripe"): rows [0, max_t_v) are the compressed tokens in the
 * same order as the V segments (2-bit rows, then 4-bit, then 8-bit, each head
 * filling a prefix), rows [max_t_v, t_k) are the tokens whose V stays fp16.
 * Per-head counts are read from device memory (v_seg_bounds, n_v16) when the
 * kernel runs, never from host copies.
 */
typedef struct rdkv_layer_view {
  const uint8_t* k2;          /* [H_kv][rows][n_ch2_pad/4] quarter-split bytes, or NULL */
  const uint8_t* k4;          /* [H_kv][rows][n_ch4_pad/2] half-split bytes, or NULL    */
  const uint8_t* k8;          /* [H_kv][rows][n_ch8], or NULL                           */
  int64_t k2_head_stride;     /* bytes between heads                                    */
  int64_t k4_head_stride;
  int64_t k8_head_stride;
  const uint16_t* k_scale;    /* fp16 [H_kv][d_pad], sorted+padded channel order        */
  const uint16_t* k_zp;       /* fp16 [H_kv][d_pad]                                     */
  const int64_t* k_perm;      /* int64 [H_kv][d_pad]: original channel of each slot     */
  int64_t k_perm_head_stride; /* elements between KV heads (g*d_pad for the per-q table)*/
  const uint8_t* v2;          /* [H_kv][rows][32] or NULL                               */
  const uint8_t* v4;          /* [H_kv][rows][64] or NULL                               */
  const uint8_t* v8;          /* [H_kv][rows][128] or NULL                              */
  int64_t v2_head_stride;     /* bytes between heads                                    */
  int64_t v4_head_stride;
  int64_t v8_head_stride;
  const uint16_t* v_scale;    /* fp16 [H_kv][v_meta_head_stride], head-local row order  */
  const uint16_t* v_zp;
  int64_t v_meta_head_stride; /* elements between heads                                 */
  const uint16_t* v16;        /* fp16 [H_kv][rows][128] Zone-B values, or NULL          */
  int64_t v16_head_stride;    /* elements between heads                                 */
  const int32_t* v_seg_bounds;/* int32 [H_kv][3] = (n2, n4, n8) per head; NULL = use    */
  int32_t n2, n4, n8;         /*   these shared counts for every head                   */
  const int32_t* n_v16;       /* int32 [H_kv] Zone-B rows per head; NULL = n_v16_shared */
  int32_t n_v16_shared;
  const float* mask;          /* optional additive fp32 [H_q][mask_row_stride] (0/-inf) */
  int64_t mask_row_stride;
  int32_t n_ch2_pad;          /* shared-max padded channel counts (multiples of 4/2/1)  */
  int32_t n_ch4_pad;
  int32_t n_ch8;
  int32_t max_t_v;            /* stripe row where Zone B starts                         */
  int32_t t_k;                /* stripe rows to attend over                             */
  int32_t reserved;
  /* Readable extent in bytes from each base pointer (0 for a NULL pointer).  The fused
   * kernel stages 16-byte-aligned ranges and never touches memory outside
   * [base, base + extent). */
  int64_t k2_bytes, k4_bytes, k8_bytes;
  int64_t v2_bytes, v4_bytes, v8_bytes, v16_bytes;
  int64_t v_meta_bytes;       /* extent of v_scale and of v_zp                          */
} rdkv_layer_view;

/* ── library ──────────────────────────────────────────────────────────────── */
int rdkv_version(void);                    /* ABI version, bumps on any signature change */
const char* rdkv_last_error_string(int status);
int rdkv_last_cuda_error(void);            /* cudaError_t of the last failed launch (this thread) */
int rdkv_sizeof_layer_view(void);          /* lets a binding check its struct layout     */

/* ── K side: scores over packed channels ─────────────────────────────────────
 * Replaces k_mixed_qk_dot_into / k_mixed_qk_dot
 * (obkv_accel/triton_k_kernel.py:1211-1427) and the Triton kernels they dispatch
 * to (:96-956).  out[h_q][t] = (sum_c code*(q[perm c]*scale c) - sum_c zp c *
 * q[perm c]*scale c) / sqrt(128) for t < t_eff; columns >= t_eff are untouched.
 * `view` is a HOST pointer (copied into the launch).  q: [H_q][128] with
 * q_row_stride elements between rows; out: fp32 with out_row_stride elements. */
int rdkv_k_scores(const rdkv_layer_view* view, const void* q, int q_dtype, int64_t q_row_stride,
                  int H_q, int H_kv, int t_eff, float* out, int64_t out_row_stride, void* stream);

/* ── V side: weighted sum over packed tokens ──────────────────────────────────
 * Replaces v_dequant_weighted_sum_dispatch[_into]
 * (obkv_accel/triton_v_kernel.py:1274-1313, 1729-1760) and kernels :131-1098.
 * out[h_q][d] = sum over the head's 2/4/8-bit rows of w[h_q][col]*(code-zp)*scale
 * (col = head-local row index) + sum over its fp16 rows of
 * w[h_q][max_t_v + j]*v16[j][d].  out is fully overwritten; summation order is
 * fixed (no atomics).  `view` is a HOST pointer. */
int rdkv_v_weighted_sum(const rdkv_layer_view* view, const float* w, int64_t w_row_stride,
                        int H_q, int H_kv, float* out, int64_t out_row_stride, void* stream);

/* ── fused split-sequence decode attention ────────────────────────────────────
 * Replaces the attention block of the decode loop
 * (obkv_accel/fast_decode.py:1701-1784: K kernel, mask add, softmax, V kernel)
 * for n_views (sequence, layer) pairs in one launch.  views: DEVICE array.
 * q: [n_views][H_q][128].  Every head's live rows (its 2-, 4-, 8-bit rows, then its
 * fp16 rows; stripe padding is skipped) are cut into chunks of chunk_rows rows;
 * chunk c of view v, query head h writes one partial record at
 * partials[((v*H_q + h)*n_chunks + c) * RDKV_PARTIAL_STRIDE] (an empty record
 * m=-inf, l=0, o=0 when the head has no row in that chunk).  n_chunks must be
 * >= ceil(max live rows / chunk_rows).  With n_chunks == 1 and out != NULL the
 * normalised result goes straight to out (fp32 [n_views][H_q][128]) and partials
 * may be NULL.  k_row_bytes_max: largest K bytes per row (sub_2 + sub_4 + n_ch_8)
 * over the views; it sizes the shared-memory stages (rdkv_decode_stage_bytes).
 * status: optional device int32, OR-ed with 1 if a staging wait ran out and with 2
 * if a view did not fit the launch (k_row_bytes_max too small, or more than 384
 * padded channels); the affected records are then invalid.
 * Alignment: V code tensors 4-byte, fp16 V tensor 8-byte, scale/zp 2-byte aligned. */
/* The two halves of the same kernel behind the reference's two-stage interface
 * (views: DEVICE array of ONE view):
 * rdkv_decode_scores — what k_mixed_qk_dot_into computes
 * (obkv_accel/triton_k_kernel.py:1211-1427): scores[h][t] for every stripe row
 * t < t_eff (rows that belong to no token hold the zero point and score 0 up to
 * rounding, as in the reference); q [H_q][128] contiguous; V is not read.
 * rdkv_decode_weighted_sum — what v_dequant_weighted_sum_dispatch_into computes
 * (obkv_accel/triton_v_kernel.py:1729-1760): out[h][:] = sum_t weights[h][t] * V^[t]
 * with weight columns = stripe rows; out fp32 [H_q][128] contiguous; K is not read;
 * unit_rows >= the longest head's live rows (one CTA per KV head, fixed summation
 * order). */
int rdkv_decode_scores(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q,
                       int H_kv, int chunk_rows, int n_chunks, int k_row_bytes_max, int t_eff,
                       float* scores, int64_t scores_row_stride, int32_t* status, void* stream);
int rdkv_decode_weighted_sum(const rdkv_layer_view* views, int n_views, int H_q, int H_kv, int unit_rows,
                             int k_row_bytes_max, const float* weights, int64_t weights_row_stride,
                             float* out, int32_t* status, void* stream);
int rdkv_decode_stage_bytes(int k_row_bytes_max);
int rdkv_decode_attn_partial(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype,
                             int H_q, int H_kv, int chunk_rows, int n_chunks, int k_row_bytes_max,
                             float* partials, float* out, int32_t* status, void* stream);

/* The uncompressed tail and the token being decoded, for rdkv_decode_attn_tail.
 * Replaces, together with the packed zones, the whole attention block of a decode step
 * (obkv_accel/fast_decode.py:1644-1784): fused_rope on q and the new k (triton_rope.py:35-108),
 * the append of the new K / V rows to the buffers of decode-generated tokens (:863-866) and one
 * softmax over Zone A | Zone B | Zone C (:1719-1784). */
typedef struct rdkv_tail_args {
  void* new_k;                   /* [n_views][H_kv][cap][128] fp16 / bf16, rows contiguous; the   */
  void* new_v;                   /*   tokens generated so far (Zone C); 16-byte aligned            */
  int64_t view_stride;           /* elements between views (multiple of 8)                          */
  int64_t head_stride;           /* elements between KV heads (multiple of 8)                       */
  int32_t dtype;                 /* RDKV_F16 or RDKV_BF16: type of new_k, new_v, k_cur, v_cur       */
  int32_t cap;                   /* rows each head's buffer holds                                   */
  int32_t n_new;                 /* live rows of every view when n_new_per_view is NULL             */
  int32_t rope_dtype;            /* type of rope_cos / rope_sin (RDKV_F16 / BF16 / F32)             */
  const int32_t* n_new_per_view; /* device int32 [n_views] (clamped to [0, cap]), or NULL           */
  const void* rope_cos;          /* [..][64] cosines / sines of the position (half format: channel  */
  const void* rope_sin;          /*   i pairs with i + 64), or NULL / NULL: q and k_cur are rotated  */
  int64_t rope_view_stride;      /* elements between views' tables (0: one table for all views)     */
  const void* k_cur;             /* [n_views][H_kv][128] key / value row of the token being decoded */
  const void* v_cur;             /*   (k_cur not yet rotated), or NULL / NULL: no such token        */
  int32_t append;                /* 1: the rotated k_cur and v_cur are also written to row n_new of */
  int32_t reserved;              /*   new_k / new_v (status bit 2 if the buffer is full)            */
} rdkv_tail_args;
int rdkv_sizeof_tail_args(void);           /* lets a binding check its struct layout */

/* The same kernel with everything a decode step needs in ONE launch (new; same reference
 * block, obkv_accel/fast_decode.py:1701-1784):
 *   - seq_part / seq_parts: the sequence split.  Part i of n takes, of every head, rows
 *     [n_p*i/n, n_p*(i+1)/n) (rounded down to multiples of 32) of each of its four V phases (its
 *     n_p 2-bit rows, its 4-bit rows, its 8-bit rows, its fp16 rows), so the parts read about the
 *     same bytes; the ranks that share a head pass their part of the same packed layer and ask
 *     for out_record (0 / 1 = everything).
 *   - row_begin / row_end: of the rows left by the part, numbered phase after phase, only
 *     [row_begin, row_end) are attended over (0 / INT32_MAX = all of them); chunk c covers rows
 *     [row_begin + c*chunk_rows, +chunk_rows) cut at row_end.
 *   - unit_recs / k_slots / nkb_max: optional prepared table of the views (rdkv_decode_prepare
 *     below); NULL / NULL / 0 = the kernel reads counts, scales, zero points and permutations from
 *     the views' own tensors (a second, dependent round trip per CTA).
 *   - n_whole_units: of the launch's units (view, KV head, group of 8 query heads; in that order)
 *     the first n_whole_units are attended over by one CTA each whatever n_chunks says; only the
 *     remaining ones are cut into n_chunks chunks.  CTAs start in launch order, so a launch whose
 *     units do not fill the last round of CTAs evenly can keep full rounds of whole units and cut
 *     just the leftover ones finely enough to fill the last round (0 = cut every unit).
 *   - n_chunks > 1: chunk records go to partials ([n_views*H_q][n_chunks][132]) and the last CTA of
 *     each (view, KV head, group of 8 query heads) to finish merges them in chunk order; nobody
 *     waits.  unit_counters: int32 [n_views][H_kv * ceil(g/8)], zero before the first launch; the
 *     kernel leaves them zero again.  Launches that share counters or partials must not overlap.
 *   - exactly one of out (normalised fp32 [n_views][H_q][128]) and out_record (un-normalised
 *     (m, l, -, -, o[128]) per (view, query head), input of rdkv_lse_combine across shards);
 *     out, out_record and partials 16-byte aligned (they are written four floats at a time). */
int rdkv_decode_attn(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q,
                     int H_kv, int chunk_rows, int n_chunks, int n_whole_units, int row_begin, int row_end,
                     int seq_part, int seq_parts, int k_row_bytes_max, const void* unit_recs, const void* k_slots, int nkb_max,
                     float* partials, int32_t* unit_counters, float* out, float* out_record,
                     int32_t* status, void* stream);

/* rdkv_decode_attn plus the uncompressed tail in the same launch and the same softmax (one more
 * tile phase of plain 16-bit K and V rows, scored on the tensor cores) and, optionally, the token
 * being decoded: its key row is rotated like the queries, scored, weighted with its value row as
 * the first term of the running softmax, and (append) written behind the tail for later steps;
 * the queries are rotated on the way in (the caller's q is not written).  chunk_rows, row_begin /
 * row_end and seq_part count the tail rows behind the fp16 rows of a head.  Always launches the
 * one-item-per-CTA form of the kernel. */
int rdkv_decode_attn_tail(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype, int H_q,
                          int H_kv, int chunk_rows, int n_chunks, int n_whole_units, int row_begin, int row_end,
                          int seq_part, int seq_parts, int k_row_bytes_max, const void* unit_recs,
                          const void* k_slots, int nkb_max, float* partials, int32_t* unit_counters,
                          float* out, float* out_record, int32_t* status, const rdkv_tail_args* tail,
                          void* stream);

/* fused_rope (obkv_accel/triton_rope.py:111-138) on its own: rotates n_q rows of q and n_k rows of
 * k (128 channels each, row strides in elements) in place with one table of 64 cosines / sines;
 * fp32 arithmetic with every product and sum rounded separately, result rounded to the rows'
 * type (bit-identical to fused_rope_ref, :141-165). */
int rdkv_rope(void* q, int q_dtype, int n_q, int64_t q_row_stride, void* k, int k_dtype, int n_k,
              int64_t k_row_stride, const void* cos_half, const void* sin_half, int cs_dtype, void* stream);

/* Persistent form of rdkv_decode_attn (same arguments and results): one resident CTA per slot
 * of the GPU goes through the launch's work items (whole units first, then chunks) in steps of the
 * grid size, its staging warp running ahead across item boundaries, so that the start-up round
 * trips and the pipeline drain are paid once per CTA instead of once per (view, KV head).
 * Requirements beyond rdkv_decode_attn's: a prepared table (unit_recs, k_slots) in which every
 * unit's byte ranges lie on whole 16-byte blocks (flag bit 0 of its record; a unit without it is
 * reported through status bit 2 and left empty), no mask in the views, q 16-byte aligned, and
 * work_counters: int32 [2], zero before the first launch (the CTAs draw their items from it and
 * the last one to finish puts it back to zero; launches that share it must not overlap). */
int rdkv_decode_attn_persistent(const rdkv_layer_view* views, int n_views, const void* q, int q_dtype,
                                int H_q, int H_kv, int chunk_rows, int n_chunks, int n_whole_units,
                                int row_begin, int row_end, int seq_part, int seq_parts,
                                int k_row_bytes_max, const void* unit_recs, const void* k_slots,
                                int nkb_max, float* partials, int32_t* unit_counters,
                                int32_t* work_counters, float* out, float* out_record, int32_t* status,
                                void* stream);

/* Prepared table of a set of views (new; the reference re-derives the same per-head quantities
 * in Python before every kernel call, obkv_accel/triton_k_kernel.py:1236-1285).  Per (view, KV
 * head): the head's V row counts (n2, n4, n8, n16), where the rows of each V phase start in every
 * tensor, a flag saying that every byte range of the head can be staged in whole 16-byte blocks,
 * and the head's kept K channels as the fused kernel's threads consume them (original channel,
 * zero point, scale per padded slot, in MMA fragment order).
 * It is a snapshot of the view records and of their count, K scale, K zero-point and permutation
 * tensors: a caller that rewrites any of those in place runs rdkv_decode_prepare again (one small launch, capturable)
 * before the next rdkv_decode_attn that is given the table.  Packed payloads and V scales / zero
 * points are never copied.
 *   nkb_max: max over the views of rdkv_decode_k_blocks(n_ch2_pad, n_ch4_pad, n_ch8) (<= 24);
 *   unit_recs: rdkv_decode_prepared_bytes(n_views*H_kv, nkb_max, 0) bytes, 16-byte aligned;
 *   k_slots:   rdkv_decode_prepared_bytes(n_views*H_kv, nkb_max, 1) bytes, 16-byte aligned.
 * A launch over a sub-range of the views starting at view v0 offsets the two pointers by
 * v0*H_kv units (rdkv_decode_prepared_bytes(1, nkb_max, 0) resp. (1, nkb_max, 1) bytes per unit). */
int rdkv_decode_k_blocks(int n_ch2_pad, int n_ch4_pad, int n_ch8);
int64_t rdkv_decode_prepared_bytes(int64_t n_units, int nkb_max, int which);
int rdkv_decode_prepare(const rdkv_layer_view* views, int n_views, int H_kv, int nkb_max, void* unit_recs,
                        void* k_slots, const void* v_maps, void* stream);
/* Tensor maps of the views' V tensors (new; no counterpart in the reference).  With them the fused
 * kernel brings a tile's V rows into shared memory as one tiled TMA box per tile whose inner extent
 * is 16 bytes wider than a row (the excess arrives as zeros), so that the rows sit 48 / 80 / 144 /
 * 272 bytes apart and the four rows a quad of threads reads together fall on distinct banks;
 * without them (v_maps == NULL, or a phase whose map could not be encoded: base not 16-byte
 * aligned, empty tensor) the staging warp places the rows at the same pitch with 16-byte copies.
 *   rdkv_decode_v_map_bytes(n_views): size of the map block, 4 maps of 128 bytes per view (2-bit,
 *     4-bit, 8-bit, fp16 rows);
 *   rdkv_decode_encode_v_maps(views_host, n_views, maps_host): HOST call: encodes the maps of
 *     n_views view records held in host memory (their v2 / v4 / v8 / v16 pointers and byte
 *     counts) into maps_host; returns the number of maps encoded (the others are all zero), or -1
 *     on bad arguments.  The caller copies the block to device memory (64-byte aligned) and hands
 *     it to rdkv_decode_prepare as v_maps, which records per (view, KV head, phase) the map and the
 *     row number of the head's first row.  The block must stay alive and unchanged as long as the
 *     table is used; a table whose V tensors move is encoded and prepared again. */
int64_t rdkv_decode_v_map_bytes(int n_views);
int rdkv_decode_encode_v_maps(const rdkv_layer_view* views_host, int n_views, void* maps_host);

/* Log-sum-exp merge of split-sequence partials (new; the reference has no
 * split path — it is the combine step of the fused call above and of the
 * multi-GPU sequence split).  For each of n_rows rows merges n_splits records
 * found at partials + (row*row_stride + s*split_stride) floats, in index order:
 * M = max m_s, L = sum l_s e^{m_s-M}, out = sum o_s e^{m_s-M} / L  (0 when L = 0).
 * out: fp32 [n_rows][128]; out_ml: optional fp32 [n_rows][2] = (M, L);
 * out_partial: optional record array [n_rows][RDKV_PARTIAL_STRIDE] holding the
 * merged but un-normalised partial (input of a further combine, e.g. across GPUs). */
int rdkv_lse_combine(const float* partials, int64_t n_rows, int n_splits, int64_t row_stride,
                     int64_t split_stride, float* out, float* out_ml, float* out_partial,
                     void* stream);

/* ── prefill: stable partition of a bit map ───────────────────────────────────
 * Replaces the argsort(stable)/nonzero bookkeeping of pack_v_segments,
 * build_packed_layer and pack_k_mixed (obkv_accel/packing.py:733-735, 898-917,
 * 240-256).  bits: [n_rows][len] integers of elem_size bytes (1,2,4,8).
 * mode 0 (tokens): classes 2,4,8,16 ; mode 1 (channels): 16 counts as 8, classes 2,4,8.
 * order[row][j]: source index of the j-th kept element in class order (class 2
 * first ... each class ascending), -1 past the kept count.  counts[row][4].
 * mode + 4: the entries past the kept count are left as they are (a caller that reads the lists
 * through counts saves the fill: 7/8 of the writes at a budget of 1/8 of the tokens). */
int rdkv_partition_by_bits(const void* bits, int elem_size, int64_t row_stride, int n_rows, int len,
                           int mode, int32_t* order, int32_t* counts, void* stream);

/* ── prefill: per-token V quantise + bit-pack ─────────────────────────────────
 * Replaces quantize_and_pack(dim=3) + transfer_8bit_to_{2,4}bit_batchwise as
 * used by pack_v_segments (obkv_accel/packing.py:141-165, 715-778;
 * obkv_accel/bitpack.py:13-40) and the per-head padding/stacking of
 * _pad_and_stack_per_head_layers (:1116-1158, 1262-1278).
 * V: fp16 [H][T][D] (v_head_stride, v_row_stride in elements).  order/counts as
 * produced by rdkv_partition_by_bits mode 0 (order_row_stride 0 = one map shared
 * by all heads; order NULL = identity over n_identity rows of class `identity_bits`).
 * Head h writes rows [0,n2_h) of out2 ([H][max_n2][D/4]), [0,n4_h) of out4
 * ([H][max_n4][D/2]), [0,n8_h) of out8 ([H][max_n8][D]), rows [0,n16_h) of out16
 * (fp16 [H][max_n16][D]) and scale/zp[h][0..t_v_h) (fp16 [H][max_t_v]); all
 * remaining rows up to the max_* extents are zero-filled.
 * quant_bits_override > 0 quantises every class to that many bits but keeps one
 * code per byte in out8 (the plain quantize_and_pack(dim=3) contract). */
int rdkv_pack_v(const uint16_t* V, int64_t v_head_stride, int64_t v_row_stride, int H, int D,
                const int32_t* order, int64_t order_row_stride, const int32_t* counts,
                int64_t counts_row_stride, int n_identity, int identity_bits,
                int max_n2, int max_n4, int max_n8, int max_n16,
                uint8_t* out2, uint8_t* out4, uint8_t* out8, uint16_t* out16,
                uint16_t* out_scale, uint16_t* out_zp, int max_t_v, int quant_bits_override,
                void* stream);

/* ── prefill: per-channel K quantise + bit-pack on the stripe ─────────────────
 * Replaces pack_k_mixed / pack_k_mixed_per_head (obkv_accel/packing.py:177-578)
 * run over the zero-padded stripe canvas that _pad_and_stack_per_head_layers
 * builds (:1186-1206), including its property that pad rows take part in the
 * per-channel min/max.
 * K: fp16 [H][T][D].  tok_order/tok_counts: token partition (mode 0) giving the
 * stripe row -> source token map (row s < t_v_h: order[s]; row max_t_v + j,
 * j < n16_h: order[t_v_h + j]; other rows are zero rows).  tok_order NULL =
 * identity over t_k rows.  ch_order/ch_counts: channel partition (mode 1).
 * Channel slot layout is [n_ch2_pad | n_ch4_pad | n_ch8]; a head's kept
 * channels fill a prefix of each block, the rest are zero columns.
 * scratch: fp32 [H][rdkv_pack_k_slabs(t_k)][2][d_pad] (per head: one block of
 * (min, max) per slab of stripe rows, then one block holding the final scale and
 * zero point in fp32).
 * Outputs: k2 [H][t_k][n_ch2_pad/4], k4 [H][t_k][n_ch4_pad/2], k8 [H][t_k][n_ch8],
 * scale/zp fp16 [H][d_pad], sort_idx int64 [H][d_kept_max] (0-padded),
 * perm int64 [H][d_pad] (pad -> 0), perm_q int64 [H*g][d_pad] or NULL,
 * seg_bounds int32 [H][3].
 * quant_bits_override > 0: quantise all kept channels with that many bits, one
 * code per byte in k8 (plain quantize_and_pack(dim=2)). */
int rdkv_pack_k_slabs(int t_k);
int rdkv_pack_k(const uint16_t* K, int64_t k_head_stride, int64_t k_row_stride, int H, int D,
                const int32_t* tok_order, int64_t tok_order_row_stride, const int32_t* tok_counts,
                int64_t tok_counts_row_stride, int max_t_v, int t_k,
                const int32_t* ch_order, int64_t ch_order_row_stride, const int32_t* ch_counts,
                int64_t ch_counts_row_stride, int n_ch2_pad, int n_ch4_pad, int n_ch8,
                int d_kept_max, int gqa, float* scratch,
                uint8_t* k2, uint8_t* k4, uint8_t* k8, uint16_t* out_scale, uint16_t* out_zp,
                int64_t* sort_idx, int64_t* perm, int64_t* perm_q, int32_t* seg_bounds,
                int quant_bits_override, void* stream);

/* ── decode: the uncompressed tail (Zone C) ───────────────────────────────────
 * Tokens appended during decoding stay as plain K / V rows (the reference's
 * new-token buffer, obkv_accel/fast_decode.py:863-866; its scores and weighted
 * sum, :1719-1784: softmax over [packed zones || tail]).  Writes one
 * (m, l, -, -, o[128]) record per (view, query head), m in natural-log units,
 * for rdkv_lse_combine to merge with the record of the packed zones.
 * new_k / new_v: [n_views][H_kv][cap][128] fp16, bf16 or fp32 with the given
 * element strides (rows 16- resp. 8-byte aligned); the first n_new rows of every
 * head are live, or n_new_per_view[view] rows when that device array is given; cap = rows each
 * head's buffer holds (counts read on the device are clamped to [0, cap]). */
int rdkv_tail_attn_partial(const void* q, int q_dtype, int64_t n_views, int H_q, int H_kv,
                           const void* new_k, const void* new_v, int kv_dtype,
                           int64_t kv_view_stride, int64_t kv_head_stride, int64_t kv_row_stride,
                           int n_new, const int32_t* n_new_per_view, int cap, float* partial, void* stream);

/* ── prefill: importance scores that feed the allocator ───────────────────────
 * Replaces _score_one_layer (obkv_fast.py:854-896) and apply_score_pooling
 * (obkv_fast.py:208-246).
 * rdkv_score_layer: aw [BH][R][T] attention weights of the observation window
 * (BH = batch x KV heads, R = query heads per KV head x window positions), q
 * [BH][R][D], k [BH][T][D] (element strides given) ->
 *   layer_token   fp32 [BH][T] = sum_r aw (rounded to aw's dtype, as the reference's
 *                                 aw.sum(...).float() is),
 *   layer_channel fp32 [BH][D] = mean_r(q^2) * mean_t(k^2).
 * One launch (plus a memset node for the arrival counters).  scratch:
 * rdkv_score_scratch_words(BH, T, D) 4-byte words = fp32 [BH][rdkv_score_chunks(T)][D]
 * partial sums of k^2, then one arrival counter per BH.
 * rdkv_score_pool: sliding-window pooling (stride 1) of `rows` rows of `len` fp32
 * scores; pool_max 0 = average, 1 = maximum; reflect 0 = zero padding with
 * kernel_size taps, 1 = reflection padding with min(kernel_size, 2*len-1) taps;
 * out_len must be len + 2*(taps/2) - taps + 1. */
/* rdkv_obs_scores: the same two scores straight from the observation window's queries and the
 * layer's keys, without the attention weights ever reaching memory.  Replaces the scoring step
 * of the prefill (obkv_fast.py:1443-1450: matmul in the model's 16-bit type, scaling, causal mask
 * of the window, softmax) together with _score_one_layer (:854-896).  q_obs: [BH*g] query heads of
 * W window positions x 128 (q_head_stride, q_row_stride in elements; KV head bh owns query heads
 * bh*g .. bh*g+g-1), k: [BH][T][128]; dtype RDKV_F16 or RDKV_BF16 for both; causal: window position
 * w sees keys <= T-W+w.  g*W <= 256.  scratch: rdkv_obs_scratch_words(BH, g, W, T) 4-byte words.
 * Three launches (row statistics, reduction, token sums); the keys are read twice.  The products run
 * on the tensor cores (tcgen05.mma into tensor memory); the operands are staged by tiled TMA when the
 * base addresses are 16-byte aligned, the strides multiples of 8 elements and W a multiple of 8, by
 * plain loads otherwise (same results).  The device code waits on mbarriers with a limit: the last
 * word of scratch, read as an int after the stream has drained, is 0 if no wait ran out (bit 0: the
 * staged operands did not arrive, bit 1: the products did not complete; the scores are then invalid). */
int64_t rdkv_obs_scratch_words(int BH, int g, int W, int T);
int rdkv_obs_scores(const void* q_obs, const void* k, int dtype, int64_t q_head_stride, int64_t q_row_stride,
                    int64_t k_head_stride, int64_t k_row_stride, int BH, int g, int W, int T, int causal,
                    float* scratch, float* layer_token, float* layer_channel, void* stream);
int rdkv_score_chunks(int T);
int64_t rdkv_score_scratch_words(int BH, int T, int D);
int rdkv_score_layer(const void* aw, int aw_dtype, const void* q, int q_dtype, const void* k, int k_dtype,
                     int64_t k_head_stride, int64_t k_row_stride, int BH, int R, int T, int D,
                     float* scratch, float* layer_token, float* layer_channel, void* stream);
int rdkv_score_pool(const float* scores, int64_t row_stride, int rows, int len, int pool_max,
                    int kernel_size, int reflect, float* out, int64_t out_row_stride, int out_len,
                    void* stream);

/* ── decode: scores of a block of generated tokens for its recompression ──────
 * Replaces _score_block and _channel_score of the blockwise decoder
 * (obkv_accel/blockwise_decode.py:756-810).  queries: [H_kv*g][Q][D] (element strides between
 * heads and between positions given), keys: [H_kv][T][D] (strides given); T <= 256, D <= 128.
 *   token_out   fp32 [H_kv][T] = sum over the head's g query heads and Q positions of
 *               softmax_t(q.k_t / sqrt(D)); causal != 0: position i sees keys t <= i (Q == T);
 *               NULL = channel statistic only;
 *   channel_out fp32 [H_kv][D] = mean_{g,Q}(q_d^2) * mean_t(k_d^2). */
int rdkv_block_scores(const void* queries, int q_dtype, int64_t q_head_stride, int64_t q_pos_stride,
                      const void* keys, int k_dtype, int64_t k_head_stride, int64_t k_row_stride,
                      int H_kv, int g, int Q, int T, int D, int causal, float* token_out,
                      float* channel_out, void* stream);

/* ── packed layer -> fp16 K, V ────────────────────────────────────────────────
 * Replaces unpack_k_mixed (obkv_accel/packing.py:581-709), unpack_v_segment (:1427-1444) and the
 * per-layer body of unpack_trizone_to_past_kv (obkv_accel/trizone_decompress.py:43-183, 247-290):
 * value = fp16((float(code) - float(zp)) * float(scale)), bit-identical to the reference.
 * `view` is a HOST pointer (copied into the launch).  k_out / v_out: fp16 [H_kv][rows_out][D] with
 * out_head_stride elements between heads; either may be NULL (that side is skipped).
 *   K: slot j of a head's sorted kept channels (2-bit | 4-bit | 8-bit, counts from
 *      k_ch_counts[h][3], or n_ch2 / n_ch4 / n_ch8 for every head when it is NULL) goes to original
 *      channel k_sort_idx[h * k_sort_idx_head_stride + j]; all other channels and rows >= view->t_k
 *      are zeros.
 *   V: rows [0, n2+n4+n8) of a head are its dequantised segments in head-local order, rows
 *      [view->max_t_v, + n_v16[h]) its fp16 Zone-B rows, every other row zeros. */
int rdkv_unpack_layer(const rdkv_layer_view* view, int H_kv, int D, const int64_t* k_sort_idx,
                      int64_t k_sort_idx_head_stride, const int32_t* k_ch_counts, int n_ch2, int n_ch4,
                      int n_ch8, uint16_t* k_out, uint16_t* v_out, int64_t out_head_stride, int rows_out,
                      void* stream);

/* ── prefill: every layer of a cache in one pass ──────────────────────────────
 * The reference packs a whole cache layer by layer (build_packed_cache,
 * obkv_accel/packing.py:1323-1421; driver loop obkv_fast.py:1098-1166); here the
 * layers' V and K passes run as three launches whose third grid dimension is the
 * layer.  One job per layer, in device memory; a job's fields have the meaning
 * of the like-named arguments of rdkv_pack_v / rdkv_pack_k.  rows2..rows16,
 * rows_meta, rows_k: rows allocated per head in the outputs (the per-layer
 * outputs may be slices of tensors that are taller than this layer needs).
 * scratch: fp32 [H][rdkv_pack_k_slabs(t_k)][2][d_pad] of the job. */
typedef struct rdkv_pack_job {
  const uint16_t* K; const uint16_t* V;               /* fp16 [H][T][D] of the layer */
  int64_t k_head_stride, k_row_stride, v_head_stride, v_row_stride;   /* elements */
  const int32_t* tok_order; const int32_t* tok_counts; /* [H][tok_order_row_stride], [H][4] */
  const int32_t* ch_order;  const int32_t* ch_counts;  /* [H][ch_order_row_stride],  [H][4] */
  int64_t tok_order_row_stride, ch_order_row_stride;
  int32_t D, gqa;
  int32_t max_n2, max_n4, max_n8, max_n16, max_t_v, t_k;
  int32_t rows2, rows4, rows8, rows16, rows_meta, rows_k;
  int32_t n_ch2_pad, n_ch4_pad, n_ch8, d_kept_max;
  uint8_t *v2, *v4, *v8; uint16_t *v16, *v_scale, *v_zp;
  uint8_t *k2, *k4, *k8; uint16_t *k_scale, *k_zp;
  int64_t *sort_idx, *perm, *perm_q; int32_t* seg_bounds;
  float* scratch;
} rdkv_pack_job;

int rdkv_sizeof_pack_job(void);
/* max_slots: max over jobs of max_n2+max_n4+max_n8+max_n16; max_t_k, max_d_pad: max over jobs.
 * k_passes: how K is packed.  1 = one pass over the kept rows (a cluster of 8 CTAs per (layer, head)
 * keeps them in shared memory between the extrema and the quantisation; head size 128, and
 * ceil(max_t_k / 8) rows of max_d_pad fp16 values must fit 200 KB, else RDKV_ERR_TOO_LARGE);
 * 3 = extrema pass, parameter pass, quantise pass (the rows are read twice); 0 = one pass where
 * it fits.  Both give the same bytes.  max_k_quads: max over jobs of n_ch2_pad/4 +
 * ceil(n_ch4_pad/4) + ceil(n_ch8/4) (what a parked row of the one-pass form holds, in 8-byte
 * units), or 0 for the bound max_d_pad/4 + 2. */
int rdkv_pack_kv_batched(const rdkv_pack_job* jobs, int n_jobs, int H, int D, int max_slots,
                         int max_t_k, int max_d_pad, int k_passes, int max_k_quads, void* stream);

/* ── prefill: batched Lagrangian bit allocator ────────────────────────────────
 * Replaces knapsack_bit_allocation_batched (knapsack_solver.py:121-248).
 * scores fp32 [n_rows][len] (row_stride elements); budget fp32 [n_rows];
 * options: n_options (<= 8) integer-valued bit costs and their distortions,
 * HOST arrays; out int64 [n_rows][len] receives the chosen bit value of every
 * unit.  scratch: fp32 [n_rows][2] + int32 [n_rows] = 3*n_rows 4-byte words.
 * len*max(option) must stay below 2^24 (exact fp32 means, as in the reference). */
int rdkv_knapsack_batched(const float* scores, int64_t row_stride, int n_rows, int len,
                          const float* budget, const float* option_bits, const float* option_eps,
                          int n_options, int max_iters, float tol, int64_t* out, void* scratch,
                          void* stream);

/* Single-row form, for any number of independent rows.  Replaces knapsack_bit_allocation
 * (knapsack_solver.py:39-118), whose arithmetic differs from the batched solver's: the multiplier
 * is bisected in double precision and enters the cost as its fp32 rounding, means and the
 * tolerance test are compared in double, lambda_hi has no floor and is doubled row by row until the
 * mean fits or it reaches 1e12.  budget: DEVICE array of doubles [n_rows]; no scratch. */
int rdkv_knapsack_rows(const float* scores, int64_t row_stride, int n_rows, int len, const double* budget,
                       const float* option_bits, const float* option_eps, int n_options, int max_iters,
                       double tol, int64_t* out, void* stream);

/* ── batched bit allocator without caller-provided scratch ────────────────────
 * No counterpart in the reference.  Same computation and arguments as
 * rdkv_knapsack_batched, minus `scratch`: the three words per row the two kernels
 * hand over to each other live in a fixed array inside the library's device image
 * (48 KiB on every GPU that loads the library, held until the process exits).  It is
 * meant for callers that may not allocate device memory where they call from — an
 * engine that froze its memory plan after warm-up, or a plugin that is given input
 * and output buffers and nothing else.  After one warm-up call per device the call
 * performs no allocation of any kind (the first call on a device makes the runtime
 * load the library's module there, which reserves device memory, and opts the
 * kernels into large shared memory if the row is longer than 48 KiB: warm up before
 * the memory plan is frozen, with a row as long as the longest that will follow).
 *   - n_rows above rdkv_knapsack_static_max_rows() (4096) is refused with
 *     RDKV_ERR_TOO_LARGE; split the batch or use rdkv_knapsack_batched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before
 *     any stream capture begins.
 *   - All calls on a device share the one array.  Every call overwrites the entries of
 *     its own rows before reading them, so nothing has to be cleared between calls, but
 *     two calls whose kernels overlap on the GPU (different streams) race: serialise them. */
int rdkv_knapsack_static_max_rows(void);
int rdkv_knapsack_batched_static(const float* scores, int64_t row_stride, int n_rows, int len,
                                 const float* budget, const float* option_bits, const float* option_eps,
                                 int n_options, int max_iters, float tol, int64_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RDKV_B200_H */
