/*
 * eppgcn_b200 -- C ABI of the B200 (sm_100a) GCN aggregation hot path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns
 * an int status (0 = EPP_OK) and never terminates the process.  Device
 * pointers are raw CUDA pointers on the current device; `stream` is a
 * `cudaStream_t` passed as `void*` (NULL = legacy default stream).  Device
 * entry points only enqueue work: they do not synchronise and they allocate
 * nothing (scratch is supplied by the caller) unless the comment says
 * otherwise.  Inputs are borrowed and never written unless marked in/out.
 *
 * Each declaration names the interface of the reference project
 * (Catriminal/EPPGCN, paths inside that project) that it stands in for.
 */
#ifndef EPPGCN_B200_H_
#define EPPGCN_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  EPP_OK = 0,
  EPP_ERR_BAD_ARG = 1,       /* null pointer, negative size, part size < 1 ...      */
  EPP_ERR_CUDA = 2,          /* a CUDA runtime call or launch failed                  */
  EPP_ERR_SCAN_TIMEOUT = 3,  /* the bounded look-back wait of a scan kernel ran out  */
  EPP_ERR_TOO_LARGE = 4,     /* a size is beyond what the entry point supports       */
  EPP_ERR_PEER_TIMEOUT = 5   /* the bounded wait for another GPU's flag ran out      */
};

/* Library version as major*10000 + minor*100 + patch. */
int eppgcn_version(void);
/* Static name of a status code. */
const char *eppgcn_status_string(int status);
/* Message of the calling thread's most recent failure ("" if none). */
const char *eppgcn_last_error(void);

/* ------------------------------------------------------------------------
 * Forward neighbour-group aggregation.
 * Replaces spmm_forward_cuda_kernel and its launch
 * (EPPGCN/GCNConv/EPPGCN_kernel.cu:150-184, :204-295), and, applied to
 * d_output, spmm_backward_cuda_kernel (:415-442, :471-545).
 *
 *   out[r][:] = sum over edges e of row r:
 *               (deg_row[r] * deg_col[col_idx[e]]) * feat[col_idx[e]][:]
 *
 * out       [num_nodes][dim] dense fp32, fully overwritten (rows without
 *           edges come back zero).
 * out       fp32 rows with a stride of out_ld floats (out_ld >= dim, or 0
 *           for a dense [num_nodes][dim] result); columns beyond dim are
 *           left untouched, so a caller can fill a column block of a wider
 *           matrix.
 * feat      fp32 rows with a stride of feat_ld floats (feat_ld >= dim).
 * row_ptr   [num_nodes+1], col_idx [row_ptr[num_nodes]]  int32 CSR.
 * deg_row / deg_col   per-vertex factors of the destination and the source
 *           side.  The reference passes one `degrees` array for both; a
 *           row-partitioned caller passes `degrees + first_row` as deg_row.
 *           deg_col may be NULL: the rows of feat then already carry their
 *           source-side factor (see eppgcn_update_scaled) and the kernel
 *           computes deg_row[r] * sum feat[col_idx[e]][:], one 32-byte sector
 *           less per edge.
 * part_ptr  [num_parts+1], part2node [num_parts]: the neighbour groups of
 *           build_part -- consecutive, non-overlapping, covering every row.
 * part_size, dim_worker, warp_per_block: the reference's launch knobs
 *           (EPPGCN/param.py:80-124).  Accepted for signature parity; the
 *           result does not depend on them.
 */
int eppgcn_spmm_forward(float *out, long long out_ld, const float *feat, long long feat_ld,
                        const int *row_ptr, const int *col_idx,
                        const float *deg_row, const float *deg_col,
                        const int *part_ptr, const int *part2node,
                        int num_nodes, int dim, int num_parts,
                        int part_size, int dim_worker, int warp_per_block,
                        void *stream);

/* ------------------------------------------------------------------------
 * Backward aggregation over the prepared execution path.
 * Replaces ours_backward_cuda_kernel and its launch
 * (EPPGCN/GCNConv/EPPGCN_kernel.cu:562-589, :626-670).
 *
 *   d_in[r][:] = sum over compacted edges e with ids[e] == r:
 *                (deg_row[r] * deg_col[edge_list[e]]) * d_out[edge_list[e]][:]
 *
 * d_in      [num_nodes][dim] fp32 with a row stride of d_in_ld floats (0 =
 *           dense), columns 0..dim-1 fully overwritten (rows off the path
 *           come back zero).
 * ids, edge_list   outputs of eppgcn_compact_mask (valid prefix).
 * part_ptr  [num_parts+1] output of eppgcn_split_parts; part p covers
 *           compacted edges [part_ptr[p], part_ptr[p+1]) of one row.
 * part_size, blockx, blocky: reference knobs (EPPGCN/param.py:6-24,182-200),
 *           accepted for parity; the result does not depend on them.
 * deg_col may be NULL with the same meaning as in eppgcn_spmm_forward.
 */
int eppgcn_spmm_backward_compacted(float *d_in, long long d_in_ld, const float *d_out, long long d_out_ld,
                                   const int *ids, const int *part_ptr, const int *edge_list,
                                   const float *deg_row, const float *deg_col,
                                   int num_nodes, int dim, int num_parts,
                                   int part_size, int blockx, int blocky,
                                   void *stream);

/* ------------------------------------------------------------------------
 * Planned aggregation: the same sums as eppgcn_spmm_forward (called with
 * deg_col == NULL) and eppgcn_spmm_backward_compacted, i.e. the work of
 * spmm_forward_cuda_kernel / ours_backward_cuda_kernel
 * (EPPGCN/GCNConv/EPPGCN_kernel.cu:204-295, :626-670), from a plan that is
 * prepared once per edge list.  The reference has no such object; the plan
 * replaces the per-call zero-fill (EPPGCN_kernel.cu:150, :562) and the
 * per-group atomics (:289-293, :666-668): it re-orders the rows by their
 * number of edges and keeps its own padded copy of the edge list, so that the
 * lanes of a warp always work on rows of one length class, every row of up to
 * 64 edges is stored exactly once, and only longer rows are cleared first and
 * summed with vector atomics.
 *
 *   out[r][:] = row_scale[r] * sum over edges e of row r:  src[col_idx[e]][:]
 *
 * eppgcn_tile_plan_from_csr / _from_ids take the edge list (col_idx, device)
 * besides the row structure: row_ptr [num_rows+1] (device), or the row id of
 * every edge, `ids` (device, valid prefix of num_edges entries; the edges of a
 * row must be consecutive, rows may come in any order).  Building copies the
 * row structure to the host, sorts the rows into classes there (linear time),
 * fills the padded edge copy on the device and synchronises `stream`.  The
 * device buffer (eppgcn_tile_plan_bytes, 256-byte aligned) must outlive the
 * plan; col_idx, row_ptr and ids are not needed after the build.
 * One plan serves every row width.  eppgcn_tile_plan_info: out8 = {edges, rows,
 * padded edge slots, padded row pieces, non-empty rows, rows cleared per call,
 * rows summed with atomics (more than 64 edges), whole result cleared per call}.
 * num_sources is the number of rows of the source matrix (col_idx values are
 * below it; num_rows for a square graph); the plan remembers which of them an
 * edge names.
 * eppgcn_spmm_tiles:
 * out       rows of out_ld floats (0 = dense [rows][dim]); columns 0..dim-1 of
 *           every row are written (rows without edges come back zero).
 * src       source rows, already multiplied by their source-side factor
 *           (eppgcn_update_scaled does that for the forward,
 *           eppgcn_pack_scaled_rows for the backward); row stride src_ld a
 *           multiple of 4 floats, base 16-byte aligned.
 * row_scale destination-side factor per row id, or NULL for 1.
 *
 * eppgcn_spmm_tiles_add adds the same sums to what `out` already holds
 * (red.global.add per row, nothing is cleared): an aggregation whose edge list
 * is cut into several plans runs the first with eppgcn_spmm_tiles and the others
 * with this entry point, one after the other on a stream.  No counterpart in
 * the reference.
 *
 * eppgcn_pack_scaled_rows prepares the source of a backward aggregation, in
 * place of the per-edge degrees[...] factor of ours_backward_cuda_kernel
 * (EPPGCN_kernel.cu:660-663):  dst[r][0..dim) = scale[r] * x[r][0..dim)  into
 * rows of dst_ld floats (a multiple of 4, 16-byte aligned), only for the rows
 * the plan's edges name when `plan` is given (the other rows of dst are left
 * as they are and are never read by eppgcn_spmm_tiles with that plan).
 */
typedef struct eppgcn_tile_plan eppgcn_tile_plan;
size_t eppgcn_tile_plan_bytes(long long num_edges, int num_rows, int num_sources);
int eppgcn_tile_plan_from_csr(eppgcn_tile_plan **plan, void *dev_buf, size_t dev_bytes,
                              const int *row_ptr, const int *col_idx, int num_rows, long long num_edges,
                              int num_sources, void *stream);
int eppgcn_tile_plan_from_ids(eppgcn_tile_plan **plan, void *dev_buf, size_t dev_bytes,
                              const int *ids, const int *col_idx, long long num_edges, int num_rows,
                              int num_sources, void *stream);
void eppgcn_tile_plan_destroy(eppgcn_tile_plan *plan);
int eppgcn_tile_plan_info(const eppgcn_tile_plan *plan, long long *out8);
/* The rows that have at least one edge, ascending (device int32 inside the plan's buffer). */
int eppgcn_tile_plan_active_rows(const eppgcn_tile_plan *plan, const int **rows_dev, int *count);
int eppgcn_spmm_tiles(float *out, long long out_ld, const float *src, long long src_ld,
                      const eppgcn_tile_plan *plan, const float *row_scale, int dim, void *stream);
int eppgcn_spmm_tiles_add(float *out, long long out_ld, const float *src, long long src_ld,
                          const eppgcn_tile_plan *plan, const float *row_scale, int dim, void *stream);
int eppgcn_pack_scaled_rows(float *dst, long long dst_ld, const float *x, long long ldx,
                            const float *scale, const eppgcn_tile_plan *plan, int num_rows, int dim,
                            void *stream);

/* Bounds-checking build (the library compiled with -DEPP_DEBUG_BOUNDS, see
 * eppgcn_b200/build.py): eppgcn_spmm_tiles compares every source id and row id
 * of a plan with its limit before using it; an offender is skipped, not
 * dereferenced, and the first one is recorded.  Synchronises the device and
 * returns the record {code, value, limit, tile}: code 0 = nothing found, 1 = a
 * source id beyond num_sources, 2 = a row id beyond num_rows, -1 = this is
 * not a bounds-checking build.  reset != 0 clears the record.  No counterpart
 * in the reference (its only check is cudaGetLastError + exit after a launch,
 * EPPGCN/GCNConv/EPPGCN_kernel.cu:195-199). */
int eppgcn_debug_status(int *out4, int reset);

/* ------------------------------------------------------------------------
 * Dense update of a layer with the source-side factor folded in.
 * Replaces the torch::mm(input, weight) of the forward wrapper
 * (EPPGCN/GCNConv/EPPGCN_kernel.cu:142) for narrow outputs.
 *
 *   out[r][c] = scale[r] * sum_k x[r][k] * w[k][c]        c < dout <= 32
 *
 * FP32 FMA on the CUDA cores (no reduced-precision tensor-core path).
 * x    [num_rows] rows of stride ldx floats, w [k] rows of stride ldw floats,
 * out  rows of stride ld_out floats; the call writes columns 0..dout-1 and
 *      zero-fills the pad_cols columns after them (ld_out >= dout + pad_cols).
 *      A 32-column block of a wider result is written by offsetting `out`
 *      and `w` and passing pad_cols = 0.
 * scale may be NULL (plain x @ w).  out rows must be 16-byte aligned (ld_out a
 * multiple of 4 floats); x is read fastest when ldx is a multiple of 4 too.
 * dout > 32 returns EPP_ERR_TOO_LARGE (call once per 32-column block).
 * Also used for d_input = d' @ W^T of the backward wrapper
 * (EPPGCN/GCNConv/EPPGCN_kernel.cu:614) with w = W^T.
 */
int eppgcn_update_scaled(float *out, long long ld_out, const float *x, long long ldx,
                         const float *w, long long ldw, const float *scale,
                         int num_rows, int k, int dout, int pad_cols, void *stream);

/* ------------------------------------------------------------------------
 * Weight gradient of a layer, replaces torch::mm(X.transpose(0,1), d_input_prime)
 * of the backward wrapper (EPPGCN/GCNConv/EPPGCN_kernel.cu:615).
 *
 *   dw[kk][c] = sum_r x[r][kk] * d[r][c]        dw dense [k][dout], overwritten
 *
 * FP32 FMA; partial sums of row slabs are combined with atomics, so the
 * summation order varies from run to run.  dout <= 32 and k * dout <= 4096
 * (after rounding both up to multiples of 4), else EPP_ERR_TOO_LARGE.
 * x and d must be 16-byte aligned; strides that are multiples of 4 floats are
 * read with 16-byte copies.
 */
int eppgcn_weight_grad(float *dw, const float *x, long long ldx, const float *d, long long ldd,
                       int num_rows, int k, int dout, void *stream);
/* The same product over a list of rows only,  dw = sum over i < num_listed of
 * x[rows[i]]^T d[rows[i]]  -- the masked product the reference sketches at
 * EPPGCN/GCNConv/EPPGCN_kernel.cu:607,616.  With the rows of a layer's
 * execution path (eppgcn_tile_plan_active_rows) the rows of x that face an
 * all-zero row of d are never read.  rows: device int32. */
int eppgcn_weight_grad_rows(float *dw, const float *x, long long ldx, const float *d, long long ldd,
                            const int *rows, int num_listed, int k, int dout, void *stream);

/* ------------------------------------------------------------------------
 * Execution-path marking for one preparation step.
 * Replaces mask_forward_cuda_kernel and its launch
 * (EPPGCN/GCNConv/EPPGCN_kernel.cu:311-333, :351-388).
 *
 * For every edge e of group p (row r = ids[p], column c = edge_list[e]):
 *   if (!is_last && src_mask[r + row_offset])  ngh_mask[r + row_offset] = ngh_mask[c] = 1
 *   if (src_mask[c])                           back_edge_mask[e] = r, node_degs[r] += 1
 * src_mask / ngh_mask are byte masks (torch.bool).  ngh_mask may be NULL when
 * is_last.  back_edge_mask (expected -1) and node_degs (expected 0) are
 * updated in place.  row_offset is 0 for the reference's call; a
 * row-partitioned caller passes the global id of its first row.
 */
int eppgcn_mask_forward(const int *ids, const int *part_ptr, const int *edge_list,
                        const unsigned char *src_mask, unsigned char *ngh_mask,
                        int *back_edge_mask, int *node_degs,
                        int num_parts, int is_last, int row_offset,
                        int blockx, int blocky, void *stream);

/* ------------------------------------------------------------------------
 * Stable compaction of the marked edges.
 * Replaces compact_mask -> cuCompactor_mask::compact
 * (EPPGCN/GCNConv/cuCompactor.cu:344-463, :682-686).
 *
 * Keeps, in order, every e with edge_mask[e] != -1:
 *   out_id[k] = edge_mask[e], out_edge[k] = col_idx[e]
 * and zero-fills both outputs from the kept count up to `length`.  The kept
 * count is stored to *valid_len_dev (device int).  `scratch` must hold
 * eppgcn_compact_scratch_bytes(length) bytes; the call clears what it needs.
 * `status_dev` (device int, may alias nothing else) receives EPP_OK or
 * EPP_ERR_SCAN_TIMEOUT when the kernels finish.
 * mode 0: one pass with a decoupled look-back scan (bounded wait);
 * mode 1: three kernels (tile counts, scan of counts, scatter), no waiting;
 * mode 2: self-test of the bounded wait (length > 4096): the first tile is
 *         withheld, so the look-back of the second one waits for a descriptor
 *         that never comes; the wait runs out in about a second, status_dev
 *         receives EPP_ERR_SCAN_TIMEOUT, the outputs are undefined and the
 *         context stays usable.
 */
size_t eppgcn_compact_scratch_bytes(int length);
int eppgcn_compact_mask(const int *edge_mask, const int *col_idx,
                        int *out_id, int *out_edge, int length,
                        void *scratch, size_t scratch_bytes,
                        int *valid_len_dev, int *status_dev, int mode, void *stream);

/* ------------------------------------------------------------------------
 * eppgcn_compact_mask for callers that cannot supply scratch memory.
 * Has no counterpart in the reference (which calls cudaMalloc/cudaFree inside
 * every compaction, EPPGCN/GCNConv/cuCompactor.cu:442-462).
 *
 * Same inputs, outputs and results as eppgcn_compact_mask in mode 0, but the
 * scan's tile descriptors live in a fixed array inside the library instead of
 * a caller buffer, and the call allocates nothing: no cudaMalloc, no cudaFree,
 * no allocating library routine.  Meant for hosts that must not allocate on
 * the device once they are running -- a process whose own pool already owns
 * all device memory, a thread that cannot afford the device-wide
 * synchronisation an allocation implies, an application that forbids
 * allocation after start-up.
 *
 * Limits and rules:
 *  - length <= 67,108,864 (2^26) edges; larger inputs return EPP_ERR_TOO_LARGE
 *    and must use eppgcn_compact_mask.
 *  - The array costs 131,328 bytes of device memory on every GPU that uses
 *    this library's kernels, for the life of the process.  With CUDA's default
 *    lazy module loading it comes into being when the library's module is
 *    first used on a device, not when the library file is loaded, and that
 *    first use may allocate device memory implicitly.  Make one warm-up call
 *    per device during start-up (any small input will do); calls after it
 *    allocate nothing.
 *  - The first call on a device also looks up the array's device address
 *    (once per device, with that device current).  Make that first call
 *    outside any stream capture -- the warm-up call above serves both ends.
 *  - All calls on a device share the one array.  Each call clears what it
 *    needs, so calls issued back to back on one stream are fine; two calls
 *    whose kernels can overlap on the GPU (different streams, no ordering)
 *    race on it and give undefined results.
 *  - There is no second, wait-free attempt inside the call: when *status_dev
 *    comes back as EPP_ERR_SCAN_TIMEOUT the outputs are void and the caller
 *    repeats the compaction with eppgcn_compact_mask(mode = 1), which needs
 *    caller scratch but never waits.
 */
int eppgcn_compact_mask_static(const int *edge_mask, const int *col_idx,
                               int *out_id, int *out_edge, int length,
                               int *valid_len_dev, int *status_dev, void *stream);

/* ------------------------------------------------------------------------
 * Splitting the active rows into backward parts.
 * Replaces compact_part -> cuCompactor_part::compact followed by
 * exclusive_scan (EPPGCN/GCNConv/cuCompactor.cu:492-619, :42-48, :688-692).
 *
 * For every vertex v in order with node_deg[v] > 0, ceil(deg/part_size)
 * parts; part_pointer[j] is the compacted-edge offset where part j starts and
 * part_pointer[num_parts] the total.  Entries past num_parts (up to out_len)
 * are zeroed; an entry that would land at index out_len is dropped.
 * *num_parts_dev receives the part count.  Exact for any int32 input (the
 * reference is limited to 1023 parts per vertex).  scratch/status/mode as for
 * eppgcn_compact_mask, sized by eppgcn_split_scratch_bytes(num_nodes).
 */
size_t eppgcn_split_scratch_bytes(int num_nodes);
int eppgcn_split_parts(const int *node_deg, int num_nodes, int part_size,
                       int *part_pointer, int out_len,
                       void *scratch, size_t scratch_bytes,
                       int *num_parts_dev, int *status_dev, int mode, void *stream);

/* ------------------------------------------------------------------------
 * Neighbour groups built on the device: the same partition as
 * eppgcn_build_part_host / build_part (EPPGCN/GCNConv/EPPGCN.cpp:186-227) from a
 * row pointer that already lives in device memory, in one launch (plus a
 * row-length pass), int32-exact for any offsets.  For every vertex with d > 0
 * edges, ceil(d / part_size) groups: part_ptr[g] is the group's first edge,
 * part2node[g] its vertex, part_ptr[num_parts] = row_ptr[num_nodes].
 * part_ptr_len / part2node_len are the capacities of the two outputs (entries
 * beyond them are dropped; ceil(E / part_size) + num_nodes + 1 always
 * suffices); *num_parts_dev receives the group count.  scratch / status / mode
 * as for eppgcn_split_parts, sized by eppgcn_build_part_scratch_bytes.
 */
size_t eppgcn_build_part_scratch_bytes(int num_nodes);
int eppgcn_build_part(const int *row_ptr, int num_nodes, int part_size, int *part_ptr, int part_ptr_len,
                      int *part2node, int part2node_len, void *scratch, size_t scratch_bytes,
                      int *num_parts_dev, int *status_dev, int mode, void *stream);

/* Number of non-zero entries, stored to *count_dev.
 * Replaces compact_count (EPPGCN/GCNConv/cuCompactor.cu:638-678, :694-696). */
int eppgcn_count_nonzero(const int *values, int length, int *count_dev, void *stream);

/* ------------------------------------------------------------------------
 * Row exchange between the GPUs of one node.  No counterpart in the
 * reference, which is single-GPU: these entry points serve the
 * row-partitioned aggregation, where a rank's edges reference rows that
 * other ranks own.
 *
 * eppgcn_push_rows gathers rows of this rank's matrix and stores them
 * straight into other ranks' source buffers over NVLink (plain peer stores):
 *
 *   for r in 0..world-1, for j in [send_ptr[r], send_ptr[r+1]):
 *     peer_base[r][(peer_first_row[r] + j - send_ptr[r]) * peer_ld + 0..dim)
 *         = rows[send_idx[j] * rows_ld + 0..dim)
 *
 * rows, send_idx are device pointers of the calling GPU; send_ptr [world+1],
 * peer_base [world] and peer_first_row [world] are HOST arrays; peer_base[r]
 * is rank r's buffer as mapped into this process (peer access enabled, e.g.
 * a CUDA IPC or fabric mapping), unused when rank r gets no rows.  dim,
 * rows_ld and peer_ld are multiples of 4 floats, all bases 16-byte aligned.
 * start_row (0 <= start_row < send_ptr[world]) is the send-list entry the
 * kernel begins with (it wraps around); the result does not depend on it.
 * Ranks that each start at their right-hand neighbour's rows
 * (send_ptr[(rank+1) % world]) keep every peer's NVLink ingress busy instead
 * of all storing into rank 0 first.
 * The caller orders the stores against the readers with eppgcn_peer_barrier.
 *
 * eppgcn_peer_barrier is a barrier over `world` GPUs on flag words in peer
 * memory: peer_flags [world] (HOST array) holds every rank's array of
 * `world` 32-bit words as mapped into this process, zero before the first
 * barrier.  Barrier number `value` (1, 2, 3 ... the same on all ranks)
 * stores `value` into word `rank` of every peer's array (release, system
 * scope) and waits until all words of the own array have reached it.  Work
 * enqueued before the barrier on any rank's stream is visible to work
 * enqueued after it on every rank's stream.  The wait is bounded: after
 * max_polls polls of about a microsecond each the kernel stores
 * EPP_ERR_PEER_TIMEOUT to *status_dev (device int, set to 0 by the caller
 * beforehand) and returns; the context stays usable.  While *status_dev is
 * non-zero, later barriers announce their arrival but do not wait, so a
 * broken group drains quickly; the caller reads the word and gives up.
 *
 * eppgcn_push_rows_signal is eppgcn_push_rows served peer by peer (rank-1,
 * rank-2, ... modulo world, so that every rank receives its right-hand
 * neighbour's rows first and no two ranks store into one peer at a time) with
 * a signal per peer: once all rows for peer r are stored, word `rank` of
 * peer_landed[r] (HOST array of every rank's `world`-word "landed" array as
 * mapped into this process, zero at the start) is set to *epoch_dev (release,
 * system scope).  Peers that get no rows are not signalled.  epoch_dev is a
 * device word the caller advances before every exchange (eppgcn_bump_counter,
 * on a stream that orders it before this launch and before the readers'
 * eppgcn_wait_landed launches); done_dev is scratch of
 * 16 zeroed device words that the kernel leaves zeroed.  A rank sends nothing
 * to itself: send_ptr[rank] == send_ptr[rank + 1].
 *
 * eppgcn_bump_counter adds one to a device word, in stream order.
 *
 * eppgcn_wait_landed makes the stream wait until word r of landed_dev (this
 * rank's own "landed" array) has reached *epoch_dev for every rank r whose bit
 * is set in `owners` (counters that only grow, compared modulo 2^32).  One warp
 * polls; the wait is bounded like the barrier's: after max_polls polls
 * EPP_ERR_PEER_TIMEOUT is stored to *status_dev, and while that word is
 * non-zero later waits return at once.
 *
 * eppgcn_peer_barrier_counted is the same barrier numbered on the device:
 * every launch takes the next number from *counter_dev (a 32-bit word of this
 * rank's memory, zero before the first barrier, touched by nothing else), so
 * a launch captured into a CUDA graph can be replayed.  All ranks must run the
 * same sequence of barriers on one flag array, and must not mix the two
 * numberings on it.
 */
int eppgcn_push_rows(const float *rows, long long rows_ld, const int *send_idx,
                     const long long *send_ptr, void *const *peer_base,
                     const long long *peer_first_row, long long peer_ld, int dim, int world,
                     long long start_row, void *stream);
int eppgcn_peer_barrier(void *const *peer_flags, int rank, int world, unsigned value,
                        long long max_polls, int *status_dev, void *stream);
int eppgcn_peer_barrier_counted(void *const *peer_flags, int rank, int world, unsigned *counter_dev,
                                long long max_polls, int *status_dev, void *stream);
int eppgcn_push_rows_signal(const float *rows, long long rows_ld, const int *send_idx,
                            const long long *send_ptr, void *const *peer_base,
                            const long long *peer_first_row, long long peer_ld, int dim, int world,
                            int rank, void *const *peer_landed, const unsigned *epoch_dev,
                            unsigned *done_dev, void *stream);
int eppgcn_bump_counter(unsigned *counter_dev, void *stream);
int eppgcn_wait_landed(const unsigned *landed_dev, unsigned owners, const unsigned *epoch_dev,
                       long long max_polls, int *status_dev, void *stream);

/* ------------------------------------------------------------------------
 * Host-side helpers (CPU pointers, synchronous).
 */
/* Neighbour-group partition, replaces build_part
 * (EPPGCN/GCNConv/EPPGCN.cpp:186-227).  Call with part_ptr == NULL to get
 * only *num_parts, then with part_ptr[num_parts+1], part2node[num_parts].
 * part_ptr[num_parts] is always indptr[num_nodes]. */
int eppgcn_build_part_host(int part_size, const int *indptr, int num_nodes,
                           int *part_ptr, int *part2node, long long *num_parts);
/* Regression rule of get_map_back_part_size (EPPGCN.cpp:304-310), unclamped. */
int eppgcn_map_back_part_size(int valid_node, int valid_len, int *part_size);
/* Degree-bucket rule of build_back_part (EPPGCN.cpp:243-258); leaves 0 for
 * an average degree of 512 or more, as the reference does. */
int eppgcn_bucket_back_part_size(int valid_node, int valid_len, int *part_size);
/* Ten degree-histogram features, replaces get_ginfo (EPPGCN.cpp:348-386). */
int eppgcn_get_ginfo_host(const int *node_deg, int num_nodes, int valid_len, float *out10);

/* ------------------------------------------------------------------------
 * Timers behind print_time / clear_time
 * (EPPGCN/GCNConv/EPPGCN_kernel.cu:89-116).  Events are recorded on the
 * caller's stream and resolved lazily, so timing adds no host stall per op.
 * Categories: 0 forward aggregation, 1 forward update (GEMM),
 * 2 backward aggregation (with 1-based layer), 3 backward update, 4 mask.
 */
int eppgcn_timing_enable(int on);                 /* returns previous state */
int eppgcn_time_begin(void *stream);              /* slot handle, or -1 when off */
int eppgcn_time_end(int slot, int category, int layer, void *stream);
/* Accumulated milliseconds: out[0..4] by category, out[5..10] per-layer backward aggregation. */
int eppgcn_time_read(float *out11);
int eppgcn_print_time(void);                      /* same keys and format as the reference */
int eppgcn_clear_time(void);

#ifdef __cplusplus
}
#endif
#endif /* EPPGCN_B200_H_ */
