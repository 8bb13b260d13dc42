/* f2cgt_b200 - C ABI of the B200 (sm_100a) implementation of F2CGT's compressed-feature hot path.
 *
 * This is the drop-in boundary: one `extern "C"` entry point per operator that the reference
 * (gpzlx1/F2CGT) exposes through its pybind11 module `F2CGTLib` (src/pybind.cu:7-47), plus the
 * operators its callers need that it does not bind.  The Python module `F2CGTLib` shipped with this
 * library is a thin ctypes shim over these functions.
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer unless the parameter name ends in `_host`;
 *   - tensors are dense row-major ("contiguous" in torch terms); sizes are in elements;
 *   - the library allocates nothing that outlives a call and never synchronises the device; work
 *     is queued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream,
 *     which is what the reference launches on, e.g. src/fusion_spmm.cu:261);
 *   - the return value is a status (F2C_OK = 0); on failure `f2c_last_error()` returns a message
 *     for the calling thread.  The reference aborts the process on a bad dtype
 *     (src/common.h:29,51,64,80,102) and checks nothing else; this library validates and returns;
 *   - index tensors (`indptr`, `indices`) share one dtype, int32 or int64 (the reference also
 *     instantiates int8/uint8/int16 indices, src/common.h:39-57, which no caller uses);
 *   - code tensors are uint8 / int8 / int16 (src/common.h:68-82).  Packed widths (1, 2, 4 bits)
 *     are raw bytes whatever the dtype says (src/sq_quantization.cu:131-132).
 */
#ifndef F2CGT_B200_H_
#define F2CGT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  F2C_U8 = 0, F2C_I8 = 1, F2C_I16 = 2, F2C_I32 = 3, F2C_I64 = 4, F2C_F16 = 5, F2C_F32 = 6, F2C_F64 = 7
} f2c_dtype;

typedef enum { F2C_MEAN = 0, F2C_SUM = 1 } f2c_reduce;   /* the reference only has mean */
typedef enum { F2C_L2 = 0, F2C_COSINE = 1 } f2c_metric;  /* src/kmeans.cu:16-22,107-112 */
/* f2c_kmeans_assign only: OR one of these into `metric` to pin the scorer for this call (tests, benchmarks);
 * without one the library picks by shape.  Both give the same labels. */
#define F2C_SCORER_EXACT 0x100   /* fp32 FMA scorer */
#define F2C_SCORER_TENSOR 0x200  /* tcgen05 scorer + exact re-score of undecided points (needs a workspace) */

typedef enum {
  F2C_OK = 0,
  F2C_ERR_INVALID = 1,      /* bad argument (null pointer, negative size, inconsistent shapes) */
  F2C_ERR_UNSUPPORTED = 2,  /* dtype / bit width / size outside what the library implements */
  F2C_ERR_CUDA = 3,         /* a CUDA runtime call or launch failed */
  F2C_ERR_LIMIT = 4         /* a stated size limit of the entry point was exceeded */
} f2c_status;

/* Kernel family of a fused aggregation call.  Every family computes the same bits (same decode expression, CSC
 * summation order, one division); AUTO picks the fastest one that takes the shape, the others exist so that tests and
 * benchmarks can pin one.  A pinned family that does not take the shape returns F2C_ERR_UNSUPPORTED. */
typedef enum {
  F2C_KERNEL_AUTO = 0,
  F2C_KERNEL_STREAM = 1,          /* producer warp streams neighbour data into a shared-memory ring (cp.async) */
  F2C_KERNEL_PREFETCH = 2,        /* neighbour data prefetched into registers, software-pipelined over rows */
  F2C_KERNEL_GENERAL = 3,         /* any shape: warp per destination row, arithmetic decode */
  F2C_KERNEL_PREFETCH_ARITH = 4   /* fused SQ only: the register-prefetch kernel with exp2f decode instead of the table */
} f2c_kernel;

/* Optional per-call options of the aggregation kernels: dropout fused on the aggregated output (equivalent to calling
 * f2c_dropout on the output with the same arguments) and the kernel family.  NULL = no dropout, F2C_KERNEL_AUTO. */
typedef struct {
  float p;          /* drop probability */
  int training;     /* 0 = identity */
  int scale;        /* 0 = survivors unchanged (reference, src/fusion_dropout.cu:16); 1 = times 1/(1-p) */
  uint64_t seed;    /* Philox key */
  uint64_t offset;  /* Philox stream offset (counter words 2,3) */
  int kernel;       /* f2c_kernel */
} f2c_epilogue;

const char* f2c_last_error(void);
int f2c_version(void);

/* Kernels of this library never spin without a limit: a wait that runs out (a producer warp or a tensor-core
 * barrier that does not answer within ~0.2 s) makes the kernel return early and raises a per-device word.
 * f2c_device_status synchronises `stream`, copies that word of the current device to *code_host (0 = no wait ever
 * ran out since the last query) and clears it.  Allocates nothing.  No counterpart in the reference. */
int f2c_device_status(int32_t* code_host, void* stream);

/* packbits(unpack, target_bits)  -  src/packbits.cu:44-64 (kernel :6-42).
 * unpack [rows, unpack_dim] u8 -> pack [rows, ceil(unpack_dim*bits/8)] u8; bits in {1,2,4}. */
int f2c_packbits(const uint8_t* unpack, uint8_t* pack, int64_t rows, int64_t unpack_dim, int bits,
                 void* stream);

/* unpackbits(pack, target_bits, unpack_dim)  -  src/packbits.cu:97-114 (kernel :66-95). */
int f2c_unpackbits(const uint8_t* pack, uint8_t* unpack, int64_t rows, int64_t pack_dim, int64_t unpack_dim,
                   int bits, void* stream);

/* sq_compress(src, codebooks, target_bits, column_slice)  -  src/sq_quantization.cu:65-83 (kernel
 * :5-63).  src [rows, feat_dim] f32 -> dst [rows, feat_dim] f32 holding integer-valued codes;
 * codebooks [n_codebooks, 5] f32 rows [fmin,fmax,emin,emax,mean]; bits in {1,2,4,8,16}. */
int f2c_sq_compress(const float* src, float* dst, const float* codebooks, int64_t n_codebooks, int64_t rows,
                    int64_t feat_dim, int bits, int64_t column_slice, void* stream);

/* sq_decompress(compress_data, codebooks, target_bits, column_slice, feat_dim)  -
 * src/sq_quantization.cu:158-182 (kernel :85-156).  codes [rows, src_dim] -> out [rows, feat_dim] f32. */
int f2c_sq_decompress(const void* codes, int code_dtype, const float* codebooks, int64_t n_codebooks,
                      float* out, int64_t rows, int64_t src_dim, int64_t feat_dim, int bits,
                      int64_t column_slice, void* stream);

/* vq_decompress(index_tensor, codebooks, feat_dim)  -  src/vq_quantization.cu:35-60 (kernel :5-33).
 * codes [rows, n_codebooks]; codebooks [n_codebooks, length, column_slice] f32 or f16 -> out f32. */
int f2c_vq_decompress(const void* codes, int code_dtype, const void* codebooks, int codebook_dtype,
                      float* out, int64_t rows, int64_t n_codebooks, int64_t length, int64_t column_slice,
                      int64_t feat_dim, void* stream);

/* spmm_csr(feat, indptr, indices)  -  src/fusion_spmm.cu:45-70 (kernel :13-43).  Mean (or sum) of
 * neighbour rows over a CSC block.  feat [n_src, feat_dim] f32/f16/f64 -> out [n_dst, feat_dim], same dtype. */
int f2c_spmm_csr(const void* feat, int feat_dtype, const void* indptr, const void* indices, int index_dtype,
                 void* out, int64_t n_dst, int64_t feat_dim, int reduce, void* stream);

/* Backward of spmm_csr for fp32 features (no counterpart in src/: the reference's hidden layers are DGL's SAGEConv,
 * examples/models.py:31, whose autograd does this).  grad_src [n_src, feat_dim] is zeroed, then
 * grad_src[indices[k], :] += grad_out[d, :] / max(deg(d), 1) (mean) or += grad_out[d, :] (sum) for every edge k of row d. */
int f2c_spmm_csr_backward(const float* grad_out, const void* indptr, const void* indices, int index_dtype,
                          float* grad_src, int64_t n_dst, int64_t n_src, int64_t feat_dim, int reduce, void* stream);

/* sq_decompress_spmm_csr(compress_feat, codebooks, indptr, indices, target_bit, column_slice, feat_dim)
 *  -  src/fusion_spmm.cu:240-272 (kernel :143-238).  out [n_dst, feat_dim] f32; the decoded rows are
 * never written to memory.  n_src = number of rows of `codes` (compress_feat.size(0)); every index
 * must be below it (f2c_check_csc verifies that on request). */
int f2c_sq_spmm_csr(const void* codes, int code_dtype, const float* codebooks, int64_t n_codebooks,
                    const void* indptr, const void* indices, int index_dtype, float* out, int64_t n_dst,
                    int64_t n_src, int64_t src_dim, int64_t feat_dim, int bits, int64_t column_slice, int reduce,
                    const f2c_epilogue* epilogue, void* stream);

/* The same operator over a table that is row-sharded across the GPUs of one NVSwitch box (no counterpart in
 * the reference, which keeps one host replica per machine: examples/load_dataset.py:63-85).  Row r of the table
 * is row r % rows_per_shard of shard r / rows_per_shard; shard_ptrs_host is a HOST array of `world` (<= 8)
 * device pointers, every one dereferenceable from the current device (the local shard and the other ranks'
 * shards mapped with f2c_shard_open).  The kernel reads remote rows itself with ordinary loads over NVLink: there is no
 * collective and nothing waits on another rank; the caller keeps all shards alive and unmodified during the call. */
int f2c_sq_spmm_csr_peer(const void* const* shard_ptrs_host, int world, int64_t rows_per_shard, int code_dtype,
                         const float* codebooks, int64_t n_codebooks, const void* indptr, const void* indices,
                         int index_dtype, float* out, int64_t n_dst, int64_t n_src, int64_t src_dim,
                         int64_t feat_dim, int bits, int64_t column_slice, int reduce,
                         const f2c_epilogue* epilogue, void* stream);

/* The same with the n_replicated most often sampled rows kept on EVERY GPU.  Sampling follows the degree distribution,
 * so a few per cent of the rows serve most edges (the reference caches its hottest rows per GPU the same way, ranked by a
 * presampling pass: examples/dataloader.py:234-260,273-304); the kernel then crosses NVLink only for the cold remainder.
 * Numbering: ids [0, n_replicated) are the replicated rows, read from replicated_rows (device memory of the current GPU,
 * same row layout); the sharded rows follow from id C = f2c_peer_hot_first_cold_id(n_replicated, rows_per_shard) - the
 * next multiple of rows_per_shard - so that id C + r is row r of the sharded scheme above and ONE division by
 * rows_per_shard locates either kind of row (ids between n_replicated and C are unused).  The replicated rows and the
 * shards share 16 slots of rows_per_shard ids: ceil(n_replicated / rows_per_shard) + world <= 16.  n_src = largest id + 1. */
int64_t f2c_peer_hot_first_cold_id(int64_t n_replicated, int64_t rows_per_shard);
int f2c_sq_spmm_csr_peer_hot(const void* replicated_rows, int64_t n_replicated, const void* const* shard_ptrs_host, int world,
                             int64_t rows_per_shard, int code_dtype, const float* codebooks, int64_t n_codebooks,
                             const void* indptr, const void* indices, int index_dtype, float* out, int64_t n_dst,
                             int64_t n_src, int64_t src_dim, int64_t feat_dim, int bits, int64_t column_slice, int reduce,
                             const f2c_epilogue* epilogue, void* stream);

/* Shard memory that the other ranks of the box can map (no counterpart in the reference).  These five are the only
 * entry points that allocate, free or map device memory.
 *   f2c_shard_create  allocates `bytes` on the current device, copies `rows` (device memory) into it on `stream`
 *                     (synchronised before return) and writes the 64-byte handle other processes open.
 *   f2c_shard_open    maps a handle exported by ANOTHER process into the current device's address space with peer
 *                     access; call it with the GPU that will launch the kernels as the current device.
 *   f2c_shard_close / f2c_shard_free  undo them; every consumer closes before the owner frees.
 *   f2c_shard_copy    asynchronous copy of a byte range between local memory and a mapped shard (copy engine). */
#define F2C_SHARD_HANDLE_BYTES 64
int f2c_shard_create(const void* rows, int64_t bytes, void** shard, unsigned char* handle, void* stream);
int f2c_shard_free(void* shard);
int f2c_shard_open(const unsigned char* handle, void** shard);
int f2c_shard_close(void* shard);
int f2c_shard_copy(void* dst, const void* src, int64_t bytes, void* stream);

/* vq_decompress_spmm_csr(compress_feat, codebooks, indptr, indices, feat_dim)  -
 * src/fusion_spmm.cu:107-141 (kernel :72-105).  codebooks f32 only (as in the reference, :124-134). */
int f2c_vq_spmm_csr(const void* codes, int code_dtype, const float* codebooks, const void* indptr,
                    const void* indices, int index_dtype, float* out, int64_t n_dst, int64_t n_codebooks,
                    int64_t length, int64_t column_slice, int64_t feat_dim, int reduce,
                    const f2c_epilogue* epilogue, void* stream);

/* fusion_decompress(sq_data, sq_codebooks, bits, column_slice, vq_data, vq_codebooks, feat_dim)  -
 * the operator tests/test_fusion_decompress.py:40-42 calls and defines as
 * cat(sq_decompress(sq_data), vq_decompress(vq_data)); the reference's src/ no longer has it.
 * out [sq_rows + vq_rows, feat_dim] f32, one launch. */
int f2c_hybrid_decompress(const void* sq_codes, int sq_dtype, const float* sq_codebooks, int64_t sq_n_codebooks,
                          int bits, int64_t sq_column_slice, int64_t sq_rows, int64_t sq_src_dim,
                          const void* vq_codes, int vq_dtype, const float* vq_codebooks, int64_t vq_rows,
                          int64_t vq_n_codebooks, int64_t length, int64_t vq_column_slice, float* out,
                          int64_t feat_dim, void* stream);

/* Two-level aggregation in ONE launch (no counterpart kernel in the reference, which aggregates the
 * level-2 table only: examples/conv.py:56-66, examples/compress.py:58-61).  Source row s is decoded
 * from row slot[s] of the SQ table when slot[s] >= 0 and from row s of the VQ table otherwise;
 * value = reference decode of that codec, aggregation = reference mean (src/fusion_spmm.cu:24-42).
 * slot = NULL selects HOT-FIRST NUMBERING: the graph's nodes are numbered so that the n_hot hot ones come first,
 * source row s is hot iff s < n_hot and its SQ row is row s.  That removes one random 4-byte read per edge (the
 * slot lookup) and one link of the dependent load chain; with a slot array n_hot is ignored. */
int f2c_hybrid_spmm_csr(const void* sq_codes, int sq_dtype, const float* sq_codebooks, int64_t sq_n_codebooks,
                        int bits, int64_t sq_column_slice, int64_t sq_src_dim, const void* vq_codes,
                        int vq_dtype, const float* vq_codebooks, int64_t vq_n_codebooks, int64_t length,
                        int64_t vq_column_slice, const int32_t* slot, int64_t n_hot, const void* indptr, const void* indices,
                        int index_dtype, float* out, int64_t n_dst, int64_t feat_dim, int reduce,
                        const f2c_epilogue* epilogue, void* stream);

/* The two-level aggregation (sq_shards_host != NULL) or the plain VQ aggregation (sq_shards_host == NULL, SQ arguments
 * ignored) over tables row-sharded across the GPUs of one box, like f2c_sq_spmm_csr_peer: node row r (VQ codes, slot) is
 * row r % rows_per_shard of shard r / rows_per_shard, hot row h is row h % hot_rows_per_shard of SQ shard
 * h / hot_rows_per_shard; the *_shards_host arrays are HOST arrays of `world` (<= 8) device pointers dereferenceable from
 * the current device.  slot_shards_host == NULL = hot-first numbering (node s < n_hot reads hot row s).  Served for the
 * shapes of the fast kernel (uint8 codes, 4/8/16 code bytes per row, column_slice dividing 128, 8- or 4-bit hot rows). */
int f2c_hybrid_spmm_csr_peer(const void* const* sq_shards_host, const void* const* vq_shards_host,
                             const int32_t* const* slot_shards_host, int world, int64_t rows_per_shard,
                             int64_t hot_rows_per_shard, int64_t n_rows, int64_t n_hot, int sq_dtype,
                             const float* sq_codebooks, int64_t sq_n_codebooks, int bits, int64_t sq_column_slice,
                             int64_t sq_src_dim, int vq_dtype, const float* vq_codebooks, int64_t vq_n_codebooks,
                             int64_t length, int64_t vq_column_slice, const void* indptr, const void* indices,
                             int index_dtype, float* out, int64_t n_dst, int64_t feat_dim, int reduce,
                             const f2c_epilogue* epilogue, void* stream);

/* dropout_inplace(output, p, is_training)  -  src/fusion_dropout.cu:21-29 (kernel :6-19), which the
 * reference defines but never binds.  Counter-based (Philox4x32-10) instead of a time-seeded
 * per-thread XORWOW state, so a (seed, offset) pair reproduces the mask. */
int f2c_dropout(float* x, int64_t numel, float p, int training, uint64_t seed, uint64_t offset, int scale,
                void* stream);

/* pairwise_distance(x, y, metric)  -  src/kmeans.cu:102-118 (RAFT call :114-116).
 * x [n, d], y [k, d] f32 -> dist [n, k] f32: squared L2 or cosine distance (1 - cos). */
int f2c_pairwise_distance(const float* x, const float* y, float* dist, int64_t n, int64_t k, int64_t d,
                          int metric, void* stream);

/* KMeans.predict(data)  -  src/kmeans.cu:77-98 (RAFT kmeans_predict :93-95).  labels[i] = first
 * argmin over centres of the metric above; labels are int64 as in the reference (:79-81).
 * workspace: NULL, or a device buffer of f2c_kmeans_assign_workspace(n, k, d) bytes. */
int64_t f2c_kmeans_assign_workspace(int64_t n, int64_t k, int64_t d);
int f2c_kmeans_assign(const float* x, const float* centers, int64_t* labels, int64_t n, int64_t k, int64_t d,
                      int metric, void* workspace, void* stream);

/* K-means assignment for callers that cannot allocate device memory - no counterpart in the reference.
 * Same result as f2c_kmeans_assign, but the scratch it needs is a fixed 4 MiB + 256 B array inside the library
 * (present on every GPU that loads it, until exit) instead of a caller-supplied workspace, and the call itself
 * allocates nothing.  Meant for threads inside a process whose framework allocator owns nearly all of HBM, or on
 * a latency-critical path where cudaMalloc / cudaFree would stall the device.  Limits: n <= 1,048,576 points per
 * call (F2C_ERR_LIMIT beyond), k <= 256, d <= 64.  The first call on a device looks up the array's address
 * (a synchronising runtime query).  All calls on a device share the array: calls that overlap on the GPU race. */
int f2c_kmeans_assign_static(const float* x, const float* centers, int64_t* labels, int64_t n, int64_t k, int64_t d,
                             int metric, void* stream);
/* Companion of f2c_kmeans_assign_static (no counterpart in the reference either): its caller cannot read the
 * built-in array, so this copies the array's 8-byte header to the host after `stream` has drained - the number of
 * points the exact scorer had to settle and the code the kernel writes when one of its bounded waits ran out
 * (then some labels are unwritten).  Returns F2C_ERR_CUDA when that code is non-zero.  Allocates nothing.
 * (f2c_kmeans_assign reports the same two words as int32 words 0 and 1 of the caller's workspace.) */
int f2c_kmeans_assign_static_status(int32_t* undecided_host, int32_t* error_host, void* stream);

/* Debug helper (no counterpart: the reference never checks that indices < compress_feat.size(0)).
 * Writes 0 to *flag_device if indptr is non-decreasing from 0.. and every index is in [0, n_src),
 * else a non-zero code.  Asynchronous; the caller reads the flag. */
int f2c_check_csc(const void* indptr, const void* indices, int index_dtype, int64_t n_dst, int64_t n_src,
                  int32_t* flag_device, void* stream);

/* csr_sampling(indptr, indices, seeds, num_pick, replace=False) of the reference's absent ShmTensor
 * submodule (call sites examples/dataloader.py:174-175,287-288): uniform neighbour sampling without
 * replacement.  Step 1 writes out_deg[i] = min(in_degree(seeds[i]), num_pick); the caller builds
 * out_indptr as the exclusive prefix sum of out_deg; step 2 writes the sampled GLOBAL neighbour ids of
 * seed i at out_indices[out_indptr[i] ...].  All id tensors share index_dtype.  num_pick <= 64.
 * out_capacity = 0: out_indices has exactly out_indptr[n_seeds] entries.  out_capacity > 0: out_indices has that many
 * entries (the worst case n_seeds * num_pick, so that the caller need not read the edge count back from the device);
 * the unused tail is filled with seeds[0], a valid id that a later relabelling already knows. */
int f2c_sample_degrees(const void* indptr, const void* seeds, void* out_deg, int index_dtype, int64_t n_seeds,
                       int num_pick, void* stream);
int f2c_sample_neighbors(const void* indptr, const void* indices, const void* seeds, const void* out_indptr,
                         void* out_indices, int64_t out_capacity, int index_dtype, int64_t n_seeds, int num_pick,
                         uint64_t rng_seed, uint64_t rng_offset, void* stream);

/* tensor_relabel([seeds, sub_indices]) of the reference's absent ShmTensor submodule (call sites
 * examples/dataloader.py:176-177,289-290): the distinct ids of `keys` (the concatenation, seeds first) are numbered
 * 0..n_unique-1 in order of first occurrence, so distinct seeds keep their positions.  Two steps around a prefix sum
 * the caller owns: mark writes first[i] = 1 where position i is the first occurrence of its id (building a hash table
 * of `capacity` = f2c_relabel_capacity(n) slots: table_keys 8 B, table_pos 4 B per slot); the caller computes
 * rank = exclusive prefix sum of first (same dtype as the ids) and n_unique = its total; assign writes
 * unique[rank[i]] = keys[i] at first occurrences and relabelled[i] = new number of keys[i].  *error_flag (device)
 * becomes 1 if the table overflowed (never with the advised capacity), 2 if a key is negative (ids must be >= 0:
 * -1 is the table's empty marker). */
int64_t f2c_relabel_capacity(int64_t n_keys);
int f2c_relabel_mark(const void* keys, int index_dtype, int64_t n_keys, void* table_keys, void* table_pos, int64_t capacity,
                     int32_t* first, int32_t* error_flag, void* stream);
int f2c_relabel_assign(const void* keys, int index_dtype, int64_t n_keys, const void* table_keys, const void* table_pos,
                       int64_t capacity, const int32_t* first, const void* rank, void* unique, void* relabelled,
                       void* stream);

/* One hop of a minibatch block in one call: csr_sampling followed by tensor_relabel([seeds, sub_indices]), the pair the
 * reference's loader runs per hop (examples/dataloader.py:167-182).  Same sampler, same numbering as the separate entry
 * points above; the prefix sums run inside, so the host makes one call and one read per hop.
 *   sub_indptr [n_seeds + 1]                CSC offsets of the block
 *   keys       [n_seeds * (num_pick + 1)]   seeds, then the sampled global ids; entries behind n_seeds + sub_indptr[n_seeds]
 *                                           are copies of seeds[0]
 *   unique     [n_seeds * (num_pick + 1)]   distinct ids in order of first occurrence; the first header[1] are valid
 *   relabelled [n_seeds * (num_pick + 1)]   keys rewritten to positions in unique
 *   header_device [4] (int64, device)       {edges sampled, distinct ids, relabel error flag (0 ok, 1 table overflow,
 *                                           2 negative id), 0}
 * workspace: f2c_sample_block_workspace(n_seeds, num_pick, index_dtype) bytes of device memory, 256-byte aligned. */
int64_t f2c_sample_block_workspace(int64_t n_seeds, int num_pick, int index_dtype);
int f2c_sample_block(const void* indptr, const void* indices, const void* seeds, int index_dtype, int64_t n_seeds, int num_pick,
                     uint64_t rng_seed, uint64_t rng_offset, void* sub_indptr, void* keys, void* unique, void* relabelled,
                     int64_t* header_device, void* workspace, int64_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* F2CGT_B200_H_ */
