// Launch wrappers of the plain (SIMT) kernels of the search path; definitions in kernels.cu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace certex_b200 {

enum DType : int { kF32 = 0, kF16 = 1, kI8 = 2, kU8 = 3 };
enum Metric : int { kL2 = 0, kIP = 1, kCos = 2 };

inline int dtype_size(int dt) { return dt == kF32 ? 4 : dt == kF16 ? 2 : 1; }

/// Which stored rows a query may return. Everything is optional (null = absent); a set bit keeps.
struct Admit {
  const uint8_t* removed;       // [n] non-zero = removed
  const uint32_t* bits;         // bitset (one bit per row) or bitmap (one row of bits per query) words
  int64_t bitmap_cols;          // 0: `bits` is a bitset; > 0: bitmap with this many bits per query row
  const int32_t* row_labels;    // [n]; used together with query_labels
  const int32_t* query_labels;  // [nq]
};

/// e[r] for rows [row0, row0 + n) of `vectors`: -floor(|x|^2 / 2) (L2) or 0 (inner product); removed rows and the
/// padding up to `n_pad` get kNeverInit. Integer dtypes only.
void launch_row_init(const void* vectors, size_t pitch, int dtype, int d, int metric, const uint8_t* removed,
                     int64_t row0, int64_t n, int64_t n_pad, int32_t* init, cudaStream_t s);

/// e of the anchors of the threshold stage in tile order: out[t * 256 + c] = init[(c * n_tiles + t) * stride].
/// With `bits` (a bitset over the ids, set = keep; perm: sorted row -> id) dropped anchors get `never`.
void launch_gather_init(const int32_t* init, int64_t stride, int64_t n_tiles, int32_t* out, cudaStream_t s,
                        const uint32_t* bits = nullptr, const int32_t* perm = nullptr, int32_t never = 0);

/// Smallest e of every chain of 16 columns, in the tile order of the chained anchor pass: out[t * 16 + i] = min over
/// w < 16 of init[t * stride_t + i * stride_i + w * stride_w] (strides in elements). A chain that holds a removed row
/// gets the never-value and so drops out of the thresholds.
void launch_gather_chain_min(const int32_t* init, int64_t stride_w, int64_t stride_i, int64_t stride_t, int64_t n_tiles,
                             int32_t* out, bool is_float, cudaStream_t s);

/// e[j] = never (-2^30, or -inf as float bits) where removed[j] is set, j < n.
void launch_mask_removed(int32_t* e, const uint8_t* removed, int64_t n, bool is_float, cudaStream_t s);

/// cmax[c] = max of init over rows [16c, 16c + 16), chains c0 .. c0 + n - 1 (int32 values, or float bits).
void launch_chain_max(const int32_t* init, int64_t c0, int64_t n, int32_t* cmax, bool is_float, cudaStream_t s);

/// fp16 codes of n float32 / float16 rows (natural order, rows zero padded to code_pitch) with e [n] and the running
/// maxima (|code|, |rounding residual|, |e| as float bits; [3]: a coordinate did not fit fp16). See kernels.cu.
void launch_encode_f16_rows(const void* vectors, size_t pitch, int dtype, int d, int metric, int64_t n, void* codes,
                            size_t code_pitch, float* e, unsigned int* maxima, cudaStream_t s);

/// fp16 codes of the queries and shift [nq], the per-query allowance for rounding that separates the anchors' k-th
/// group maximum from the screen's threshold; *overflow is raised when a query coordinate does not fit fp16.
void launch_encode_f16_queries(const void* queries, size_t qpitch, int dtype, int d, int64_t nq, void* codes,
                               size_t code_pitch, float n1max, float n2max, float emax, float* shift,
                               unsigned int* overflow, cudaStream_t s);

/// thr [nq] of fp16 codes. step 0: float keys of the k-th largest group maxima -> keys of (value - shift / 2), scores
/// that k rows certainly reach; step 1: such keys -> float bits of the screen's threshold (bound - shift / 2).
void launch_finish_thr_f16(int32_t* thr, const float* shift, int nq, int step, cudaStream_t s, int per = 1);

void launch_fill_i32(int32_t* p, int64_t n, int32_t v, cudaStream_t s);

/// Sorts one appended batch by squared norm and writes it into the index arrays of the integer screen: e [n] are the
/// per-row terms of ids id0 .. id0 + n - 1 (see launch_row_init), the batch occupies sorted rows row0 .. row0 + n - 1;
/// perm [row] = id, inv [id] = row, init [row] = e of that id, codes [row] = code row of that id (read from
/// src + (id - src_id0) * pitch). e holds int32 values or, with is_float, float bits. keys / ids are scratch of n
/// elements each, temp of sort_batch_temp_bytes(n).
size_t sort_batch_temp_bytes(int64_t n);
void launch_sort_batch(const int32_t* e, int64_t n, int32_t id0, int64_t row0, const void* src, int64_t src_id0, size_t pitch,
                       int metric, bool is_float, uint32_t* keys_in, uint32_t* keys_out, int32_t* ids_in, int32_t* ids_out,
                       void* temp, size_t temp_bytes, void* codes, int32_t* perm, int32_t* inv, int32_t* init, cudaStream_t s);

/// Survivor records of the screen (see make_record) -> cnt [nq] / cand [nq, cap]; rows >= n_rows are dropped, rows are
/// translated to ids through perm (when not null).
void launch_expand_records(const uint64_t* rec, const unsigned long long* rec_count, unsigned long long rec_cap,
                           int64_t n_rows, const int32_t* perm, uint32_t* cnt, int32_t* cand, uint32_t cap, int sm_count,
                           cudaStream_t s);

/// thr[q] = k-th largest of gmax[q, 0:ng]  (INT_MIN when ng < k). With ng_rows [nq] every row has its own length
/// (at most ng); a negative length gives thr[q] = never. With topk [nq, k] the k largest values of every row are
/// written there too (any order: the values above the k-th, then copies of it), in the same launch.
void launch_kth_largest(const int32_t* gmax, int64_t ld, int ng, int k, int nq, int32_t* thr, cudaStream_t s,
                        const int32_t* ng_rows = nullptr, int32_t never = 0x7fffffff, int32_t* topk = nullptr);

/// thr[q] = the k-th largest of the union of parts[p, q, 0:k], p < n_parts (lists of the k largest keys of every row
/// shard: every key is reached by a row of its own, so the k-th largest of all of them is reached by k rows of the
/// whole set). scratch: nq * round_up(n_parts * k, 8) ints.
void launch_union_kth(const int32_t* parts, int n_parts, int nq, int k, int32_t* scratch, int32_t* thr, cudaStream_t s);

/// order [n] = the partition entries by (label, norm): inside a label the rows sorted by their term e of the screen
/// (stable: equal norms keep ascending ids). keys_in / keys_out: scratch of n; temp of label_norm_order_temp_bytes(n).
size_t label_norm_order_temp_bytes(int64_t n);
void launch_label_norm_order(const int32_t* part_ids, int64_t n, const int32_t* labels_of_ids, const int32_t* inv,
                             const int32_t* init, bool is_float, unsigned long long* keys_in, unsigned long long* keys_out,
                             int32_t* order, void* temp, size_t temp_bytes, cudaStream_t s);

/// Label-ordered layout of the partition (see label_rows_kernel in kernels.cu).
void launch_label_rows(const int32_t* part_ids, int64_t n, const int64_t* off, const int64_t* lrow0, int n_labels,
                       const int32_t* inv, const int32_t* init, int32_t* lperm, int32_t* linv, int32_t* lsrc, int32_t* linit,
                       cudaStream_t s);

/// Marks ids as removed: removed[id] = 1, and for the integer screen init[inv[id]] = kNeverInit with the chain maxima
/// of the touched chains recomputed; *n_new counts first-time removals.
void launch_remove(const int64_t* ids, int64_t n_ids, int64_t size, uint8_t* removed, int32_t* init, const int32_t* inv,
                   int32_t* cmax, bool is_float, unsigned long long* n_new, cudaStream_t s);

/// Optional second output of launch_verify_select for queries whose candidate list is incomplete: a tighter threshold
/// from the k-th best exact score among the candidates that were listed. thr2 is written at the query's position in
/// ovf_list; thr [nq] are the thresholds of the pass that produced the candidates; kind 1: integer values, 2: fp16
/// codes (shift [queries of the call] = the rounding allowance, see launch_encode_f16_queries). thr2 == null: off.
struct Refine {
  int32_t* thr2;
  const int32_t* thr;
  const float* shift;
  int kind;
};

/// out [n_pad, out_pitch] = rows sel[0 .. n) of `in` (row_bytes each, zero padded; sel null: rows 0 .. n - 1; a negative
/// entry: a zero row); rows n .. n_pad - 1 are zeros.
void launch_gather_rows(const void* in, size_t in_pitch, const int32_t* sel, int64_t n, int64_t n_pad, void* out,
                        size_t out_pitch, size_t row_bytes, cudaStream_t s);
/// best_s / best_row rows sel[i] = rows i of s2 / row2, i < n (negative sel[i]: skipped).
void launch_scatter_best(const double* s2, const int32_t* row2, const int32_t* sel, int n, int k, double* best_s,
                         int32_t* best_row, cudaStream_t s);
/// list[i] = sel[list[i]] for i < *n (at most n_max).
void launch_compose(int32_t* list, const unsigned int* n, int n_max, const int32_t* sel, cudaStream_t s);

/**
 * Exact fp64 scores of every query's candidate rows, then its k best by (score, row). One block per query.
 * cand [nq, cap] rows, cnt [nq] how many (a query with cnt > cap is skipped and its index appended to ovf_list;
 * so is every query when *rec_count > rec_cap, i.e. when the screen's survivor records did not all fit).
 * best_s / best_row [nq, k] (row -1, score +inf where fewer than k admitted candidates exist).
 * `where` (8-bit rows only, optional): `vectors` is not in id order, row where[id] of it holds the vector with that id
 * (the norm-sorted code rows of an index whose vectors live in host memory).
 */
void launch_verify_select(const void* vectors, size_t pitch, int dtype, int d, int metric, const void* queries,
                          size_t qpitch, int nq, int q0, const int32_t* cand, const uint32_t* cnt, uint32_t cap, int k,
                          Admit adm, double* best_s, int32_t* best_row, int32_t* ovf_list, unsigned int* ovf_count,
                          unsigned long long* stats, const unsigned long long* rec_count, unsigned long long rec_cap,
                          Refine rf, cudaStream_t s, const int32_t* where = nullptr, const double* sqnorm = nullptr);

/// out[r] = |x_r|^2 of n float32 / float16 rows, summed over the coordinates in order in fp64 with every product and sum
/// rounded on its own: the sum the cosine verification makes per candidate. With it (sqnorm of launch_verify_select,
/// indexed by row id) the verification of the cosine metric leaves that sum out.
void launch_row_sqnorms(const void* vectors, size_t pitch, int dtype, int d, int64_t n, double* out, cudaStream_t s);

/// Limits of one launch_dense_scores call: four queries of d doubles sit in shared memory (32 d bytes of the 227 KB a
/// block may have), and the queries of a call are the second grid dimension in fours.
constexpr int kDenseMaxDim     = 7264;
constexpr int kDenseMaxQueries = 4 * 65535;

/// All-pairs exact fp64 scores of queries qsel[0:nqb] (or q0.. when qsel is null) against rows [0, n): out [nqb, ld].
/// Rows that `adm` rejects score +inf. d <= kDenseMaxDim, nqb <= kDenseMaxQueries.
void launch_dense_scores(const void* vectors, size_t pitch, int dtype, int d, int metric, int64_t n, const void* queries,
                         size_t qpitch, const int32_t* qsel, int q0, int nqb, Admit adm, double* out, int64_t ld,
                         cudaStream_t s);

/// k best (score, row) of every row of scores [nqb, ld] (n valid columns); writes result row qsel[i] (or q0 + i).
/// Long rows are selected from in select_topk_parts(n, k) chunks by separate blocks and merged; part_s / part_row are
/// scratch of nqb * parts * k elements (unused when parts == 1).
int select_topk_parts(int64_t n, int k);
void launch_select_topk(const double* scores, int64_t ld, int64_t n, int k, const int32_t* qsel, int q0, int nqb,
                        double* best_s, int32_t* best_row, double* part_s, int32_t* part_row, cudaStream_t s);

/// One label's share of a search by labels: queries order[q_begin .. q_begin + nq) against the n_part partition entries
/// part_ids[part_off ..] followed by the rows added after the partition. Its scores are nq rows of ld doubles from
/// score_off; blk_begin is the first block of the group in the scoring launch.
struct LabelGroup {
  int32_t q_begin;
  int32_t nq;
  int64_t part_off;
  int32_t n_part;
  int32_t ld;
  int64_t score_off;
  int64_t blk_begin;
};

/// Blocks the scoring launch spends on a group of nq queries and n_cols columns.
int64_t grouped_blocks(int nq, int64_t n_cols);

/// Exact fp64 scores of every group (rows `adm` rejects score +inf); n_blocks = sum of grouped_blocks over the groups.
void launch_dense_scores_grouped(const void* vectors, size_t pitch, int dtype, int d, int metric, const void* queries,
                                 size_t qpitch, const int32_t* order, const LabelGroup* groups, int n_groups,
                                 int64_t n_blocks, const int32_t* part_ids, int64_t tail0, int64_t n_tail, Admit adm,
                                 double* out, cudaStream_t s);

/// launch_select_topk over ragged score rows: row i starts at scores + row_off[i], has row_n[i] <= n_max columns and
/// answers query qsel[i]. part_s / part_row: nqb * select_topk_parts(n_max, k) * k elements.
void launch_select_topk_ragged(const double* scores, const int64_t* row_off, const int32_t* row_n, int64_t n_max, int k,
                               const int32_t* qsel, int nqb, double* best_s, int32_t* best_row, double* part_s,
                               int32_t* part_row, cudaStream_t s);

/// best_row of the queries of every group: column of the group's score row -> id.
void launch_group_columns_to_ids(int32_t* best_row, int k, const int32_t* order, const LabelGroup* groups, int n_groups,
                                 const int32_t* part_ids, int64_t tail0, cudaStream_t s);

/// Label partition: part_ids = ids 0 .. n - 1 in (label, id) order, distinct / counts = the distinct labels ascending
/// and how many rows carry each, *n_distinct their number. labels_sorted, ids_in: scratch of n; distinct, counts: n.
size_t label_partition_temp_bytes(int64_t n);
void launch_label_partition(const int32_t* labels, int64_t n, int32_t* labels_sorted, int32_t* ids_in, int32_t* part_ids,
                            int32_t* distinct, int32_t* counts, int32_t* n_distinct, void* temp, size_t temp_bytes,
                            cudaStream_t s);

/// neighbors / distances / (optional) fp64 scores of the public result from the internal best lists.
/// id = row < 0 ? -1 : id_base + row. Distances: L2 s, inner product (|q|^2 - s) / 2, cosine s / 2.
void launch_finish(const double* best_s, const int32_t* best_row, int64_t id_base, const void* queries, size_t qpitch,
                   int dtype, int d, int metric, int nq, int k, int64_t* neighbors, float* distances, double* scores_out,
                   cudaStream_t s);

/// Merge of `parts` answer lists per query, [parts, nq, k] (score, id) with id -1 = missing, by (score, id);
/// writes merged ids, fp64 scores and float distances. part_stride: elements between the lists of consecutive parts
/// (0: nq * k, densely packed). With finish = false only the merged ids and fp64 scores are written (an intermediate
/// round of a merge of more candidates than one block sorts).
void launch_merge(const double* in_s, const int64_t* in_id, int parts, int nq, int k, const void* queries, size_t qpitch,
                  int dtype, int d, int metric, int64_t* neighbors, float* distances, double* scores_out, cudaStream_t s,
                  int64_t part_stride = 0, bool finish = true);

/// *status = 1 if a candidate list of the call overflowed, + 2 if a pass gave up on a wait, + 4 if a query coordinate
/// did not fit fp16 (count: the call's counters, see Index::search_begin).
void launch_search_status(const unsigned int* count, const unsigned int* q_ovf, unsigned long long* status, cudaStream_t s);

}  // namespace certex_b200
