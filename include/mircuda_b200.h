/*
 * C ABI of libmircuda_b200.so — the sm_100a (B200) implementation of mircuda's
 * quantized-matmul hot path.
 *
 * Every function below is `extern "C"`, takes plain pointers and sizes, and returns an
 * `int` status unless noted: 0 = success, -1 = invalid argument (including "executed on a
 * stream other than the plan's"), -2 = host allocation failure, -3 = the kernel reported a
 * bounded wait that ran out on an earlier launch of this plan, anything else = a raw
 * cudaError_t / CUresult. `stream` is a raw CUstream / cudaStream_t and must not be null.
 *
 * Plan-style operations keep the reference's contract: a plan is bound to the stream it
 * was created on; `execute` only enqueues work (no host synchronisation, no allocation);
 * operand buffers are caller-owned device memory and are not retained; a plan may be used
 * by one thread at a time.
 *
 * Each declaration cites the reference interface it replaces (path inside the reference
 * project : line). Entry points marked NEW have no counterpart there.
 */
#ifndef MIRCUDA_B200_H
#define MIRCUDA_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Library identification: (major << 16) | (minor << 8) | patch. NEW. */
uint32_t mircuda_b200_version(void);

/* Replaces `mircuda_cutlass_version` (sys/native/cutlass_probe.cu:16; declared in
 * sys/src/lib.rs:33-44), which the crate's `cutlass` feature links unconditionally. No
 * CUTLASS is linked here: the value is the release the reference pins
 * (sys/build/sources.rs:8, v4.4.2 -> 40402), i.e. the plans this library stands in for. */
unsigned int mircuda_cutlass_version(void);

/* ------------------------------------------------------------------ MXFP8 quantizer ----
 * bf16 [rows, columns] -> E4M3 codes [rows, columns] + one E8M0 scale per 32 columns,
 * written straight into the 128x4-swizzled scale layout (`scales` must be zero-filled
 * once by the caller; only real slots are written). columns % 32 == 0.
 * Replaces the run-time-compiled kernel `mircuda_mxfp8_quantize_bf16`
 * (kernels/mxfp8.cu:69-96) together with its launch in src/mxfp8/tensor_core.rs:140-158;
 * an ahead-of-time launcher because the launch geometry differs from the reference's.
 */
int mircuda_b200_mxfp8_quantize_bf16(const void* input, void* output, void* scales,
                                     uint32_t rows, uint32_t columns, void* stream);

/* The same quantizer reading its input as column blocks stored one after another: block b is a
 * contiguous [rows, block_columns] bf16 matrix with columns b * block_columns .. of every row,
 * the rank-major layout an all-gather of column shards produces (no reference counterpart).
 * Codes and scales come out exactly as for the row-major input. block_columns % 8 == 0 and
 * columns % block_columns == 0. */
int mircuda_b200_mxfp8_quantize_bf16_blocks(const void* input, void* output, void* scales,
                                            uint32_t rows, uint32_t columns,
                                            uint32_t block_columns, void* stream);

/* Row-major [rows, columns] E8M0 scales -> swizzled padded layout (one-time weight prep).
 * Replaces `mircuda_mxfp8_swizzle_scales` (kernels/mxfp8.cu:98-109) and its launch in
 * src/mxfp8/tensor_core.rs:89-107. `output` must be zero-filled by the caller. */
int mircuda_b200_mxfp8_swizzle_scales(const void* input, void* output, uint32_t rows,
                                      uint32_t columns, void* stream);

/* --------------------------------------------------------- MXFP8 block-scaled GEMM ----
 * C[m,n] (bf16) = A[m,k] (E4M3) . B[n,k]^T (E4M3), one UE8M0 scale per 32 K-elements of
 * each operand in the swizzled layout, fp32 accumulation. k % 128 == 0.
 * Replaces sys/native/mxfp8_sm120.cu:110-164, declared in
 * sys/src/platform/cutlass/mxfp8.rs:11-30. */
int mircuda_mxfp8_tc_create(int m, int n, int k, void* stream, void** output);
size_t mircuda_mxfp8_tc_workspace_bytes(const void* plan);
int mircuda_mxfp8_tc_execute(void* plan, void* stream, const void* a, const void* a_scales,
                             const void* b, const void* b_scales, void* c);
void mircuda_mxfp8_tc_destroy(void* plan);

/* NEW (diagnostic): proves the failure path of the bounded waits without disturbing the GPU.
 * Enqueues a one-warp kernel that waits 2 ms on a barrier nothing arrives at; the wait runs
 * out, the kernel returns by itself and raises the plan's status word exactly as a GEMM
 * kernel whose wait ran out would, so every later `execute` of this plan returns -3. The
 * plan is unusable afterwards (destroy it). */
int mircuda_b200_mxfp8_tc_wait_probe(void* plan, void* stream);

/* The same GEMM fused with the all-gather of a column-sharded linear. NEW (the reference is
 * single-GPU). The plan's n is this GPU's shard width; instead of a local C the epilogue
 * stores every tile into the full-width output [m, row_stride] of each of `output_count`
 * GPUs (<= 8, the caller's own buffer among them) at column `column_offset`, through
 * peer-mapped device pointers (CUDA IPC / symmetric memory), with plain stores over NVLink.
 * If `multicast_output` is not null it must be the NVSwitch multicast address of those same
 * buffers; every piece is then written once with a multimem store and replicated by the
 * switch. The caller orders the peers' reads after this launch (a cross-GPU barrier on the
 * stream). Needs m > 128 and n, row_stride, column_offset multiples of 8; -1 otherwise. */
int mircuda_b200_mxfp8_tc_execute_gather(void* plan, void* stream, const void* a,
                                         const void* a_scales, const void* b,
                                         const void* b_scales, void* const* outputs,
                                         int output_count, int row_stride, int column_offset,
                                         void* multicast_output);

/* All-gather of column blocks with the copy engines, the alternative to the gather epilogue
 * above for linears sharded along N (no reference counterpart: the reference is single-GPU).
 * Every rank holds a full-width [rows, pitch] output in peer-mapped memory (`buffers[p]` is rank
 * p's, `buffers[rank]` the caller's own) and has written its own column block of it on `stream`.
 * `send` issues one strided device-to-device copy per peer, on a stream per peer, ordered after
 * the work `stream` holds at the call; `stream` itself goes on at once. `join` makes `stream` wait
 * for every copy sent so far; the caller then synchronises the ranks before the gathered outputs
 * are read or a block is written again. With rows == 1 or width == pitch the block is contiguous
 * (the rank-major layout of an all-gather: rank r's [rows, local columns] matrix at block r of
 * every buffer) and is sent as a 1-D copy. world 2..8. `destroy` drains the copy streams. */
int mircuda_b200_column_gather_create(uint32_t world, uint32_t rank, void** gather);
int mircuda_b200_column_gather_send(void* gather, void* const* buffers, uint64_t pitch_bytes,
                                    uint64_t offset_bytes, uint64_t width_bytes, uint64_t rows,
                                    void* stream);
int mircuda_b200_column_gather_join(void* gather, void* stream);
void mircuda_b200_column_gather_destroy(void* gather);

/* Weight-only MXFP8 (bf16 activations, row-major [n, k/32] E8M0 scales, weights as
 * little-endian u32 words), any token count. Replaces `mircuda_mxfp8_bf16` and
 * `mircuda_mxfp8_bf16_tiled` (kernels/mxfp8.cu:111-217) with their launches in
 * src/mxfp8/matmul.rs:131-157. input_features % 32 == 0. Up to 8 tokens with
 * input_features % 128 == 0 and output_features % 16 == 0 run on the tensor cores with the
 * activations converted to f16 (exact for magnitudes from 2^-14 to 65504, saturating above;
 * MIRCUDA_B200_MXFP8_WEIGHT_ONLY=simt keeps the fp32 kernel, which has no such limit). */
int mircuda_b200_mxfp8_bf16(const void* input, const void* weight, const void* scales,
                            void* output, uint32_t tokens, uint32_t input_features,
                            uint32_t output_features, void* stream);

/* ---------------------------------------------------------- NVFP4 block-scaled GEMM ----
 * C[m,n] (bf16) = alpha * A[m,k] (E2M1) . B[n,k]^T (E2M1), one UE4M3 scale per 16 K-elements
 * of each operand in the swizzled layout, fp32 accumulation. k % 64 == 0.
 * Replaces sys/native/fp4_sm120.cu:110-170, declared in
 * sys/src/platform/cutlass/fp4/mod.rs:15-35. */
int mircuda_fp4_create(int m, int n, int k, void* stream, void** output);
size_t mircuda_fp4_workspace_bytes(const void* plan);
int mircuda_fp4_execute(void* plan, void* stream, const void* a, const void* a_scales,
                        const void* b, const void* b_scales, void* c, float alpha);
void mircuda_fp4_destroy(void* plan);

/* ----------------------------------------------------------- FP4 x FP4 GEMV (M = 1) ----
 * y[n] (bf16) = alpha * sum_k e2m1(x) e2m1(W) sx sw; k % 64 == 0.
 * Replaces sys/native/fp4_vector_sm120.cu:127-168, declared in
 * sys/src/platform/cutlass/fp4/vector.rs:11-29. With n % 128 == 0 and k % 2048 == 0 launches
 * overlap as described for mircuda_b200_nvfp4_vector_* below (weights and weight scales are
 * fetched early; MIRCUDA_B200_OVERLAP_LAUNCHES=0 serialises). execute returns -3 after a
 * launch whose bounded wait ran out. */
int mircuda_fp4_vector_create(int n, int k, void* stream, void** output);
int mircuda_fp4_vector_execute(void* plan, void* stream, const void* input,
                               const void* input_scales, const void* weight,
                               const void* weight_scales, void* output, float alpha);
void mircuda_fp4_vector_destroy(void* plan);

/* The same FP4 x FP4 GEMV without a plan and without any allocation. This entry point has
 * no counterpart in the reference. It is for hosts that do not allow this library to call
 * the CUDA allocator (all device memory already belongs to the host's own arena, or the
 * caller only owns raw pointers inside someone else's pool): the cross-slice scratch that
 * mircuda_fp4_vector_create would allocate lives in a fixed 1 MiB + 4 KiB device array inside
 * the library instead, which every GPU that loads the library holds until the process ends.
 * Limits: ceil(k / 512) * ceil(n / 128) * 128 <= 262144 and n <= 131072; a larger shape
 * returns -4 and launches nothing. The first call on each device looks up the array's
 * device address (with that device current); make that first call outside any stream
 * capture. All calls on a device share the one array: it keeps the previous call's contents
 * (the call clears the part that must start at zero), and two calls whose kernels overlap
 * on the GPU, e.g. on different streams, race. */
int mircuda_b200_fp4_vector_execute_static(int n, int k, void* stream, const void* input,
                                           const void* input_scales, const void* weight,
                                           const void* weight_scales, void* output, float alpha);

/* ------------------------------------------------------------ dense GEMV (M = 1) ----
 * y = alpha W x + beta y, data_type 0 = f16, 1 = bf16, fp32 accumulation.
 * Replaces sys/native/dense_vector_sm120.cu:147-175, declared in
 * sys/src/platform/cutlass/dense/vector.rs:14-32. */
int mircuda_dense_vector_create(int data_type, int n, int k, void* stream, void** output);
int mircuda_dense_vector_execute(void* plan, void* stream, const void* input, const void* weight,
                                 void* output, float alpha, float beta);
void mircuda_dense_vector_destroy(void* plan);

/* ------------------------------------------- bf16-activation x NVFP4-weight GEMV ----
 * y[m,n] (bf16) = global_scale * sum_k x[m,k] e2m1(W[n,k]) ue4m3(sw[n,k/16]), m <= 8.
 * NEW: the decode shape the benchmark configuration names; the reference serves it
 * through its Marlin NVFP4 dense path (src/marlin/execute.rs:109-128), whose numerics
 * (fp32 accumulation, global scale applied before the bf16 round) this follows.
 * Weights and scales use the same layouts as mircuda_fp4_vector_*. k % 64 == 0.
 * Launch overlap: for shapes with n % 128 == 0 and k % 2048 == 0 (the streaming kernel) a launch
 * may start fetching `weight` and `weight_scales` while earlier work on the stream is still
 * running (programmatic dependent launch); `input` is read and `output` written only after
 * that work has completed. Weights and scales must therefore not be written by work still in
 * flight on the stream when `execute` is called (they are model constants). The environment
 * variable MIRCUDA_B200_OVERLAP_LAUNCHES=0, read at plan creation, restores fully serialised
 * launches. */
int mircuda_b200_nvfp4_vector_create(int m, int n, int k, void* stream, void** output);
int mircuda_b200_nvfp4_vector_execute(void* plan, void* stream, const void* input,
                                      const void* weight, const void* weight_scales,
                                      void* output, float global_scale);
void mircuda_b200_nvfp4_vector_destroy(void* plan);

/* Routed weight-only MXFP8 projection (bf16 activations, MoE decode): assignment a uses input
 * row a / selections_per_input and matrix selected[a] of weight [matrices, rows, columns]
 * (E4M3 bytes, row-major E8M0 scales [matrices, rows, columns/32], optional bf16 bias
 * [matrices, rows], null for none); an out-of-range matrix writes zeros. Replaces
 * `mircuda_mxfp8_bf16_gathered` (kernels/mxfp8.cu:219-271) and its launch in
 * src/mxfp8/gathered.rs. columns % 32 == 0, assignments <= 65535. */
int mircuda_b200_mxfp8_bf16_gathered(const void* input, const void* weight, const void* scales,
                                     const void* bias, const void* selected, void* output,
                                     uint32_t assignments, uint32_t matrices, uint32_t rows,
                                     uint32_t columns, uint32_t selections_per_input,
                                     void* stream);
/* MXFP8 embedding lookup: output[t, :] = bf16(e4m3(W[row]) * 2^(s - 127) * output_scale) for
 * row = selected[selected_start + t]; rows >= vocab leave their output row untouched. Bit-
 * identical to `mircuda_mxfp8_embedding_bf16` (kernels/mxfp8.cu:273-296), which it replaces.
 * hidden % 32 == 0, tokens <= 65535. */
int mircuda_b200_mxfp8_embedding_bf16(const void* weight, const void* scales,
                                      const void* selected, void* output,
                                      uint32_t selected_start, uint32_t tokens, uint32_t vocab,
                                      uint32_t hidden, float output_scale, void* stream);

/* bf16 [rows, k] -> NVFP4 codes [rows, k/2] + swizzled UE4M3 scales per 16, given the
 * tensor's global scale (amax / 2688) in device memory. NEW: the reference has no NVFP4
 * quantizer. `mircuda_b200_nvfp4_global_scale` computes that scale into *global_scale
 * (a device float; also usable as the GEMV's global when read back). k % 64 == 0. */
int mircuda_b200_nvfp4_global_scale(const void* input, size_t elements, void* global_scale,
                                    void* stream);
int mircuda_b200_nvfp4_quantize_bf16(const void* input, const void* global_scale, void* codes,
                                     void* scales, uint32_t rows, uint32_t k, void* stream);
/* The same quantizer with the scales left row-major, [rows, k/16] bytes, for rows that are
 * moved (dispatched to another GPU) before their final place and scale tile are known;
 * mircuda_b200_mxfp8_swizzle_scales (a plain byte permutation) then builds the atoms. */
int mircuda_b200_nvfp4_quantize_rows_bf16(const void* input, const void* global_scale,
                                          void* codes, void* row_scales, uint32_t rows,
                                          uint32_t k, void* stream);

/* -------------------------------------------------- variable-row grouped bf16 GEMM ----
 * For each group g: C[off_g : off_g + min(rows_g, max_rows), :] = A[same rows] . W_g^T
 * (+ beta C); A [capacity, k], W [groups, n, k], C [capacity, n], all bf16; rows/offsets
 * are device u32 arrays that the host never reads. n % 8 == 0, k % 8 == 0.
 * Replaces sys/native/variable_grouped_bf16_sm120.cu:147-185, declared in
 * sys/src/platform/cutlass/variable_grouped/bf16.rs:11-31. */
int mircuda_variable_grouped_bf16_create(int groups, int max_rows, int n, int k, void* stream,
                                         void** output);
int mircuda_variable_grouped_bf16_execute(void* plan, void* stream, const void* input,
                                          const void* weights, const unsigned int* rows,
                                          const unsigned int* offsets, void* output, float beta);
void mircuda_variable_grouped_bf16_destroy(void* plan);
/* The same product with the weight matrix of group g picked by indices[g] out of a bank
 * W [matrices, n, k] (groups with an index >= matrices are skipped): expert-parallel MoE
 * receives one group per (source GPU, local expert). NEW: the reference's bf16 grouped plan
 * has no index array (its NVFP4 one does); plans are destroyed with
 * mircuda_variable_grouped_bf16_destroy. */
int mircuda_b200_variable_grouped_bf16_create_indexed(int groups, int matrices, int max_rows,
                                                      int n, int k, void* stream, void** output);
int mircuda_b200_variable_grouped_bf16_execute_indexed(void* plan, void* stream, const void* input,
                                                       const void* weights,
                                                       const unsigned int* indices,
                                                       const unsigned int* rows,
                                                       const unsigned int* offsets, void* output,
                                                       float beta);

/* ------------------------------------------------------- grouped NVFP4 GEMMs (MoE) ----
 * For each group g with matrix j = indices[g] (a group whose j >= matrices is skipped):
 *   C[off_g + r, :] = bf16(alphas[j] * A[off_g + r, :] . B_j^T),  r < min(rows[g], max_m)
 * A [capacity, k/2] and B [matrices, n, k/2] hold E2M1 pairs (even k low); scales are
 * swizzled UE4M3 bytes per 16 K-elements: B's per matrix with stride
 * ceil(n/128)*128 * (k/16) bytes, A's per group starting at 128-row tile
 * scale_offsets[g] / 128. All routing arrays are device u32 that the host never reads.
 * k % 64 == 0. Replace sys/native/variable_grouped_fp4_sm120.cu:178-222 and the paired
 * variant, declared in sys/native/variable_grouped_fp4_sm120.cuh:99-122. */
int mircuda_variable_grouped_fp4_create(int groups, int matrices, int max_m, int n, int k,
                                        void* stream, void** output);
int mircuda_variable_grouped_fp4_execute(void* plan, void* stream, const void* a,
                                         const void* a_scales, const void* b,
                                         const void* b_scales, const void* alphas,
                                         const unsigned int* indices, const unsigned int* rows,
                                         const unsigned int* offsets,
                                         const unsigned int* scale_offsets, void* c);
void mircuda_variable_grouped_fp4_destroy(void* plan);
/* NEW: the same product with the MoE activation fused into its epilogue. The plan's matrices are
 * gate_up banks [2 I, k] whose rows interleave gate and up in runs of 16 (rows 32 b .. 32 b + 15 =
 * gate rows 16 b .., rows 32 b + 16 .. 32 b + 31 = the up rows of the same columns; n = 2 I,
 * n % 32 == 0). Instead of bf16 C it writes what the next grouped product reads: the E2M1 codes
 * [capacity, I / 2] and swizzled UE4M3 scales (rows as in C) of bf16(silu(gate) * up) quantised
 * with the device-resident tensor scale *global_scale; bit for bit the result of the plain
 * execute on a [gate rows | up rows] bank followed by mircuda_b200_moe_swiglu_nvfp4. It removes
 * one launch and the round trip of the [capacity, 2 I] bf16 intermediate through HBM (the
 * fusion seam after the grouped plan of src/cutlass/variable_grouped/fp4/mod.rs:106-161). */
int mircuda_b200_variable_grouped_fp4_execute_swiglu(
    void* plan, void* stream, const void* a, const void* a_scales, const void* b,
    const void* b_scales, const void* alphas, const unsigned int* indices, const unsigned int* rows,
    const unsigned int* offsets, const unsigned int* scale_offsets, const void* global_scale,
    void* codes, void* scales);
/* Two such problems (left, right) that share indices / rows / offsets / scale_offsets. */
int mircuda_paired_variable_grouped_fp4_create(int groups, int matrices, int max_m, int n, int k,
                                               void* stream, void** output);
int mircuda_paired_variable_grouped_fp4_execute(
    void* plan, void* stream, const void* left_a, const void* left_a_scales, const void* left_b,
    const void* left_b_scales, const void* left_alphas, const void* right_a,
    const void* right_a_scales, const void* right_b, const void* right_b_scales,
    const void* right_alphas, const unsigned int* indices, const unsigned int* rows,
    const unsigned int* offsets, const unsigned int* scale_offsets, void* left_c, void* right_c);
void mircuda_paired_variable_grouped_fp4_destroy(void* plan);
/* Fixed m rows per group (decode): group g multiplies A rows [g*m, g*m + m) (rows [0, m) of
 * the single input when broadcast_input) by matrix selected[g] into C rows [g*m, g*m + m);
 * A scales per input group with stride ceil(m/128)*128 * (k/16) bytes. Replaces
 * sys/native/grouped_fp4_sm120.cu:145-207, declared in grouped_fp4_sm120.cuh:98-107. */
int mircuda_grouped_fp4_create(int groups, int experts, int m, int n, int k,
                               bool broadcast_input, void* stream, void** output);
int mircuda_grouped_fp4_execute(void* plan, void* stream, const void* a, const void* a_scales,
                                const void* b, const void* b_scales, const void* alphas,
                                const unsigned int* selected, void* c);
void mircuda_grouped_fp4_destroy(void* plan);

/* ----------------------------------------------- MoE row helpers around the grouped GEMMs ----
 * NEW (callers' side of the path; the reference has no counterpart). bf16 rows, columns % 8 == 0,
 * 16-byte aligned buffers, all index arrays device i32 that the host never reads.
 *   scatter_rows: destination[destination_index[i], :] = source[source_index[i], :] for i < count
 *                 (a negative source index writes zeros, a negative destination skips the item)
 *   swiglu:       output[r, j] = silu(input[r, j]) * input[r, intermediate + j], input [rows, 2*intermediate];
 *                 when row_bound is not null only the first min(rows, *row_bound) rows (device u32)
 *   combine_rows: output[t, :] = sum_j weights[t*top_k + j] * rows[index[t*top_k + j], :] (fp32 sums;
 *                 a negative index drops the term) */
int mircuda_b200_moe_scatter_rows_bf16(const void* source, const int* source_index,
                                       const int* destination_index, void* destination,
                                       uint32_t count, uint32_t columns, void* stream);
int mircuda_b200_moe_swiglu_bf16(const void* input, void* output, uint32_t rows,
                                 const unsigned int* row_bound, uint32_t intermediate,
                                 void* stream);
int mircuda_b200_moe_combine_rows_bf16(const void* rows, const int* index, const float* weights,
                                       void* output, uint32_t tokens, uint32_t top_k,
                                       uint32_t columns, void* stream);
/* Received per-group row counts [blocks * per_block] -> the rows[] / offsets[] arrays of the
 * grouped plans: group g of block s starts at s * block_rows + the `align`-rounded counts of
 * the groups before it in the block (align 128 keeps NVFP4 scale tiles per group). */
int mircuda_b200_moe_group_offsets(const int* counts, unsigned int* rows, unsigned int* offsets,
                                   uint32_t blocks, uint32_t per_block, uint32_t block_rows,
                                   uint32_t align, void* stream);

/* Expert parallelism over NVLink peer memory (NEW; no reference counterpart). Experts are
 * sharded contiguously (experts / world per GPU); an owner stores each expert's rows from all
 * sources contiguously, sources in rank order, every expert starting on a multiple of `align`
 * rows (128 for NVFP4 activations). Rows are 2-byte units here: packed codes or scale bytes
 * travel through the same kernels as `columns` = bytes / 2. all_counts [world][experts] holds every rank's
 * rows per expert (exchanged by the caller). expert_layout writes base_for_me[e] = row on e's
 * owner where this rank's rows for e start, and rows[] / offsets[] of this rank's own experts
 * for the grouped plans (and their total in *received_rows when not null). dispatch_rows copies row source_index[i] of `source` to row
 * base_for_me[sorted_expert[i]] + position[i] of the owner's receive buffer
 * (receive_buffers[owner], peer-mapped pointers; world <= 8) and records that row in
 * remote_row[i]. collect_rows sums, for every token, weights[t, j] * (row remote_row[slot[t, j]]
 * of the owner's result buffer). The caller orders these launches against the peers with its
 * own barriers; no kernel here waits for another GPU. */
/* Capacity: every rank's receive and result buffers hold `capacity_rows` rows (the same on
 * all ranks). Routing decides at run time how many rows an owner receives, so the bound is
 * enforced on the device: expert_layout clamps rows[] / offsets[] / *received_rows to it and
 * sets *overflow (a device-visible word, may be null) to 1 on every rank that sees an expert
 * run past it; dispatch_rows does not send a row at or past it and records -1 for it;
 * collect_rows adds nothing for a row recorded as -1. No access leaves the buffers; the
 * caller turns a raised word into an error. */
int mircuda_b200_moe_expert_layout(const int* all_counts, uint32_t world, uint32_t rank,
                                   uint32_t experts, uint32_t align, int* base_for_me,
                                   unsigned int* rows, unsigned int* offsets,
                                   unsigned int* received_rows, uint32_t capacity_rows,
                                   unsigned int* overflow, void* stream);
int mircuda_b200_moe_dispatch_rows_bf16(const void* source, const int* source_index,
                                        const int* sorted_expert, const int* position,
                                        const int* base_for_me, void* const* receive_buffers,
                                        uint32_t world, int* remote_row, uint32_t count,
                                        uint32_t local_experts, uint32_t columns,
                                        uint32_t capacity_rows, void* stream);
/* Row-major scale bytes [rows, columns] (as dispatched) -> the 128-row x 4-column atoms the
 * block-scaled plans read, for the first min(rows, *row_bound) rows (row_bound may be null);
 * columns % 16 == 0. Same permutation as mircuda_b200_mxfp8_swizzle_scales, 16 bytes a thread. */
int mircuda_b200_moe_scale_atoms(const void* row_scales, void* atoms, uint32_t rows,
                                 const unsigned int* row_bound, uint32_t columns, void* stream);
/* SwiGLU fused with the NVFP4 quantiser: input [rows, 2*intermediate] bf16 (gate then up),
 * outputs the codes [rows, intermediate/2] and swizzled scales of bf16(silu(gate) * up) for a
 * given (device) global scale, without writing the activated tensor; identical, bit for bit,
 * to mircuda_b200_moe_swiglu_bf16 followed by mircuda_b200_nvfp4_quantize_bf16. */
int mircuda_b200_moe_swiglu_nvfp4(const void* input, const void* global_scale, void* codes,
                                  void* scales, uint32_t rows, const unsigned int* row_bound,
                                  uint32_t intermediate, void* stream);
int mircuda_b200_moe_collect_rows_bf16(void* const* result_buffers, uint32_t world, const int* slot,
                                       const int* sorted_expert, const int* remote_row,
                                       const float* weights, void* output, uint32_t tokens,
                                       uint32_t top_k, uint32_t local_experts, uint32_t columns,
                                       void* stream);

/* ------------------------------------------------- Marlin-layout W4A16: routed (MoE) ----
 * For every assignment id = token * top_k + choice routed to expert e:
 *   output[id, :] = bf16(input[id / top_k, :] . W_e^T * scale_e) (* routing[id] if multiply_routing)
 * with weights / scales from the mircuda_marlin_* preparation entry points and routes from
 * mircuda_marlin_prepare_moe_routes (block size 8 for thread_config 0-2, 64 for 3-5).
 * `temporary`, `locks`, `atomic_reduce` are accepted for compatibility and not used (no K
 * slicing). Replace sys/native/marlin/moe_kernel.cu:175-205 and mxfp4_moe_kernel.cu:145-171,
 * declared in sys/src/platform/marlin/execute/mod.rs:32-53 and execute/mxfp4.rs:13-34.
 * output_features % 64 == 0; input_features % 16 == 0 (32 for MXFP4). Shapes with
 * input_features % 256 == 0 and <= 2048 run on a streaming kernel that converts the activations
 * bf16 -> f16 (saturating at +-65504); it reads nothing before the kernel in front of it on the
 * stream has completed. Returns -3 on every call after a launch whose bounded wait ran out. */
int mircuda_marlin_nvfp4_moe_execute(void* stream, const void* input, const void* weight,
                                     void* output, void* temporary, const void* scales,
                                     const void* global_scales, const void* sorted,
                                     const void* expert_ids, const void* padded,
                                     const void* routing, int top_k, bool multiply_routing,
                                     int tokens, int output_features, int input_features,
                                     int thread_config, void* locks, bool atomic_reduce);
int mircuda_marlin_mxfp4_moe_execute(void* stream, const void* input, const void* weight,
                                     void* output, void* temporary, const void* scales,
                                     const void* sorted, const void* expert_ids,
                                     const void* padded, const void* routing, int top_k,
                                     bool multiply_routing, int tokens, int output_features,
                                     int input_features, int thread_config, void* locks,
                                     bool atomic_reduce);

/* ------------------------------------------------------- blockwise-scaled FP8 GEMV ----
 * y[n] = bf16(sum_b input_scales[b] * weight_scales[n/128 + b * (n/128)] * sum_{k in block b}
 * e4m3(x[k]) * e4m3(W[n, k])), 128-element K blocks, fp32 scales; n % 128 == 0, k % 128 == 0.
 * Replaces sys/native/fp8_vector_sm120.cu:92-142, declared in
 * sys/src/platform/cutlass/fp8_vector.rs. workspace_bytes is always 0. */
int mircuda_fp8_vector_create(int n, int k, void* stream, void** output);
size_t mircuda_fp8_vector_workspace_bytes(const void* plan);
int mircuda_fp8_vector_execute(void* plan, void* stream, const void* input,
                               const void* input_scales, const void* weight,
                               const void* weight_scales, void* output);
void mircuda_fp8_vector_destroy(void* plan);

/* ------------------------------- FP8 matmul with token / channel scales and bias ----
 * y[m, n] = bf16(input_scales[m] * (weight_scale * sum_k e4m3(x[m, k]) * e4m3(w[n, k])) + bias[n]),
 * fp32 accumulation; the product with the weight scale is rounded to fp32 first, the rest is
 * one fma (one multiply without a bias). input_scales: m fp32. weight_scales: fp32
 * (scale_type 0) or bf16 (1); one value (weight_scale_type 0) or n (1). bias: n bf16, or null
 * when has_bias == 0. n % 16 == 0, k % 16 == 0. tile (0 or 1) selects between the reference's
 * two decode tile shapes; it is validated and otherwise has no meaning here. m <= 16 streams
 * the weights through mma.sync e4m3; larger m runs tcgen05 kind::f8f6f4.
 * Replaces sys/native/scaled_fp8_sm120.cu:125-206, declared in
 * sys/src/platform/cutlass/scaled_fp8.rs:11-36. workspace_bytes is always 0. */
int mircuda_scaled_fp8_create(int m, int n, int k, int scale_type, int weight_scale_type,
                              int has_bias, int tile, void* stream, void** output);
size_t mircuda_scaled_fp8_workspace_bytes(const void* plan);
int mircuda_scaled_fp8_execute(void* plan, void* stream, const void* input, const void* weight,
                               const float* input_scales, const void* weight_scales,
                               const void* bias, void* output);
void mircuda_scaled_fp8_destroy(void* plan);

/* ------------------------------------------------------------- dense f16 / bf16 GEMM ----
 * C[m, n] = alpha * A[m, k] . B[n, k]^T + beta * C; input_type 0 = f16, 1 = bf16; output_type
 * = input_type or 2 (f32). Any shape: k and n multiples of 8 run on tcgen05, others on a
 * CUDA-core kernel. Replaces sys/native/dense_sm120.cu:130-184, declared in
 * sys/src/platform/cutlass/dense/mod.rs:14-33. workspace_bytes is always 0. */
int mircuda_dense_create(int input_type, int output_type, int m, int n, int k, void* stream,
                         void** output);
size_t mircuda_dense_workspace_bytes(const void* plan);
int mircuda_dense_execute(void* plan, void* stream, const void* a, const void* b, void* c,
                          float alpha, float beta);
void mircuda_dense_destroy(void* plan);

/* ------------------------------------------------ W4A16 with symmetric int4 weights ----
 * NEW: the reference's W4A16 is the NVFP4/MXFP4 Marlin path; it has no int4 entry point.
 * y[m, n] = f16(sum_k x[m, k] * (q[n, k] - 8) * s[n, k / 128]): x, y f16; weights [n, k/2]
 * bytes, even k in the low nibble, q in 0..15; scales f16 [n, k/128]. k % 128 == 0,
 * n % 8 == 0. m <= 16 streams the packed weights once (HBM-bound GEMV); larger m runs a tcgen05
 * GEMM that expands the packed weights inside the kernel (the plan owns fp32 partial sums,
 * workspace_bytes, only where it splits K because m and n give few tiles;
 * MIRCUDA_B200_W4A16_PREFILL=expand selects the older form: expansion into a plan-owned f16
 * workspace of n * k halves, then the dense GEMM). At m <= 16
 * with n % 16 == 0 and k % 2048 == 0 (the streaming kernel; `scales` must then be 4-byte
 * aligned) launches overlap as described for mircuda_b200_nvfp4_vector_*: weights and scales
 * are fetched while earlier work of the stream may still run. */
int mircuda_b200_w4a16_create(int m, int n, int k, void* stream, void** output);
size_t mircuda_b200_w4a16_workspace_bytes(const void* plan);
int mircuda_b200_w4a16_execute(void* plan, void* stream, const void* input, const void* weight,
                               const void* scales, void* output);
void mircuda_b200_w4a16_destroy(void* plan);

/* ------------------------------------------------- Marlin-layout W4A16: preparation ----
 * One-time layout conversions and per-step route bucketing; stateless, integer, bit-exact.
 * Replace sys/native/marlin/repack.cu:271-end, declared in
 * sys/src/platform/marlin/prepare/mod.rs:12-42, prepare/mxfp4.rs and execute/mod.rs:18-31.
 * size_n % 64 == 0, size_k % 16 == 0 (32 for MXFP4 scales). `maximum` is a caller-owned
 * device u32 scratch; `sorted` holds assignments + experts * (block_size - 1) entries. */
int mircuda_marlin_nvfp4_repack(void* stream, const void* input, void* output, int experts,
                                int size_n, int size_k);
int mircuda_marlin_nvfp4_repack_pair(void* stream, const void* left, const void* right,
                                     void* output, int experts, int size_n, int size_k);
int mircuda_marlin_mxfp4_repack(void* stream, const void* input, void* output, int experts,
                                int size_n, int size_k, int logical_n, int logical_k,
                                bool interleaved_gate_up);
int mircuda_marlin_mxfp4_prepare_scales(void* stream, const void* input, void* output,
                                        int experts, int size_n, int size_k, int logical_n,
                                        int logical_k, bool interleaved_gate_up);
int mircuda_marlin_nvfp4_prepare_scales(void* stream, const void* left, const void* right,
                                        const void* globals, void* output, void* output_globals,
                                        void* maximum, int experts, int size_n, int size_k);
int mircuda_marlin_prepare_moe_routes(void* stream, const void* selected, const void* routing,
                                      void* sorted, void* expert_ids, void* padded, void* offsets,
                                      void* routing_f32, int assignments, int experts,
                                      int block_size);

/* --------------------------------------------------- Marlin-layout W4A16: execution ----
 * bf16 activations [tokens <= 16, k] x NVFP4 weights in Marlin tiles (prepared above) ->
 * bf16 [tokens, n]; fp32 accumulation, prepared global scale applied before the bf16 round.
 * `temporary` (>= SMs * 4096 floats) and `locks` (>= SMs ints, zero on entry, left zero)
 * are the caller-owned reduction workspace of the reference interface; `thread_config` and
 * `atomic_reduce` are accepted and ignored (one tile geometry, ordered reduction).
 * Replaces sys/native/marlin/dense_kernel.cu:73-102, declared in
 * sys/src/platform/marlin/execute/dense.rs:16-31. n % 64 == 0, k % 16 == 0.
 * Shapes with k % 512 == 0 (weights 16-byte, scales 8-byte, `temporary` 16-byte aligned) run on
 * a streaming kernel that converts the activations bf16 -> f16 (saturating at +-65504) and is
 * launched so that it may overlap the tail of the previous kernel on the stream: it reads
 * `weight` and `scales` before that kernel has completed, everything else after; a kernel that
 * writes the prepared weights must therefore not be the one directly before this call
 * (MIRCUDA_B200_OVERLAP_LAUNCHES=0 serialises the launch, MIRCUDA_B200_MARLIN_DENSE=tiles keeps
 * the tile kernel for every shape). Returns -3 on every call after a launch whose bounded wait
 * ran out. */
int mircuda_marlin_nvfp4_dense_execute(void* stream, const void* input, const void* weight,
                                       void* output, void* temporary, const void* scales,
                                       const float* global_scale, int tokens,
                                       int output_features, int input_features,
                                       int thread_config, void* locks, bool atomic_reduce);

#ifdef __cplusplus
}
#endif

#endif /* MIRCUDA_B200_H */
