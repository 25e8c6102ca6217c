/*
 * neuzip_b200 - C ABI of the B200 (sm_100a) NeuZip codec library.
 *
 * Every entry point takes raw device pointers and sizes, enqueues its work on
 * the CUDA stream passed by the caller (a cudaStream_t cast to void*; NULL is
 * the legacy default stream) and returns an int status: 0 on success, a
 * negative NZ_E_* code otherwise, with a text in nz_last_error().  The library
 * owns no tensor memory and never terminates the process.  Unless stated
 * otherwise a call does not synchronise with the host.
 *
 * "Reference" citations name files of BorealisAI/neuzip, whose native side is
 * the pybind11 module neuzip._cuda (cuda/neuzip.cu:19-106); the functions here
 * are what a binding for that module's Manager_f{precision}_n0 classes calls.
 *
 * Vocabulary.  precision s in {0,1,3,7} = mantissa bits kept.  A bf16 tensor
 * of N elements is stored as
 *   - a packed "fraction" stream of ceil(N*(s+1)/8) bytes (sign + s mantissa
 *     bits per element, MSB first), and
 *   - an NZR1 container holding the rANS-coded stream of N exponent bytes.
 * The container format is specified in oracle/nz_oracle.c.
 */
#ifndef NEUZIP_B200_H_
#define NEUZIP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NZ_OK 0
#define NZ_E_ARG (-1)      /* invalid argument (precision, size, alignment, null) */
#define NZ_E_CUDA (-2)     /* a CUDA runtime call failed */
#define NZ_E_CAPACITY (-3) /* an output or scratch buffer is too small */
#define NZ_E_FORMAT (-4)   /* malformed container */
#define NZ_E_DEVICE (-5)   /* the current device is not sm_100 */

/* Bits set by the decode kernels in the caller's 32-bit device status word. */
#define NZ_STATUS_BAD_HEADER 0x1u  /* magic / version / sizes do not match    */
#define NZ_STATUS_BAD_OFFSETS 0x2u /* unit offsets out of range / not monotone */
#define NZ_STATUS_BAD_LANES 0x4u   /* lane lengths inconsistent with the unit  */
#define NZ_STATUS_BAD_STATE 0x8u   /* a lane did not end in the initial state  */
#define NZ_STATUS_TIMEOUT 0x10u    /* a bounded wait on a bulk copy ran out    */
#define NZ_STATUS_BAD_UNIT 0x20u   /* a unit number of a gather list is out of range */

/* Library version (major*10000 + minor*100 + patch). */
int nz_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char *nz_last_error(void);

/* 0 when the current CUDA device can run the kernels (compute capability
 * 10.x), NZ_E_DEVICE otherwise.  The kernels are built for sm_100a only. */
int nz_device_check(void);

/* ---- sizes ------------------------------------------------------------- */

/* Bytes of the packed fraction stream: ceil(N*(s+1)/8).
 * Reference: cuda/high_level.cu:81-83. */
uint64_t nz_frac_bytes(uint64_t n, int precision);

/* Symbols per lane stream the library picks for a precision. */
uint32_t nz_default_lane_symbols(int precision);

/* Upper bound of the container size for n exponent bytes.
 * Reference: nvcomp CompressionConfig::max_compressed_buffer_size,
 * cuda/high_level.cu:103-108. */
uint64_t nz_container_bound(uint64_t n, uint32_t lane_symbols);

/* Bytes of device scratch nz_encode_exponents needs. */
uint64_t nz_encode_scratch_bytes(uint64_t n, uint32_t lane_symbols);

/* Bytes of device scratch nz_compress_bf16 needs (tables and one slot per coded
 * unit; the exponent stream is never written to memory). */
uint64_t nz_compress_scratch_bytes(uint64_t n, uint32_t lane_symbols);

/* ---- split / merge ------------------------------------------------------ */

/* bf16[N] -> exponent bytes u8[N] + packed fractions, with the reference's
 * round-half-up of the magnitude at the cut and carry into the exponent.
 * Reference: kernel_aligned_split, cuda/kernels.cuh:53-156 (normalized=false),
 * launched at cuda/high_level.cu:95-101 and :289-296. */
int nz_split_bf16(const void *in_bf16, uint64_t n, int precision, void *exp_out,
                  void *frac_out, void *stream);

/* Inverse of nz_split_bf16 on an uncompressed exponent stream; dropped
 * mantissa bits are zero.  canonical_nan != 0 writes 0x7FFF for every NaN
 * pattern, as the float->bf16 store of the reference does.
 * Reference: kernel_aligned_merge, cuda/kernels.cuh:158-217. */
int nz_merge_bf16(const void *exp_in, const void *frac_in, uint64_t n,
                  int precision, int canonical_nan, void *out_bf16,
                  void *stream);

/* ---- block normaliser (normalizer_size > 0) ------------------------------ */

/* Bytes of the normaliser stream: ceil(n / group), one byte per group of
 * `group` consecutive elements (a power of two up to 1024).
 * Reference: cuda/high_level.cu:89-93. */
uint64_t nz_normalizer_bytes(uint64_t n, uint32_t group);

/* Scale every group by 1.<mantissa of its absmax> before the split:
 * out = bf16(float(in) / scale), normalizers[g] = top 8 mantissa bits.
 * Reference: normalized=true path of kernel_aligned_split,
 * cuda/kernels.cuh:94-118 (intended semantics, see nz_normalize.cu). */
int nz_normalize_bf16(const void *in_bf16, uint64_t n, uint32_t group,
                      void *out_bf16, void *normalizers, void *stream);

/* Undo the scaling after the merge, in place: v = bf16(scale8 * float(v)) with
 * the scale rebuilt from the stored byte.
 * Reference: cuda/kernels.cuh:188-191, :208-216. */
int nz_denormalize_bf16(void *inout_bf16, uint64_t n, uint32_t group,
                        const void *normalizers, void *stream);

/* ---- entropy stage ------------------------------------------------------ */

/* 256-bin histogram of n bytes into hist_u32[256] (device; cleared first). */
int nz_histogram_u8(const void *sym, uint64_t n, void *hist_u32, void *stream);

/* rANS-encode n exponent bytes into an NZR1 container (device buffer of at
 * least nz_container_bound bytes, 16-byte aligned).  `scratch` is device
 * memory of nz_encode_scratch_bytes bytes, 16-byte aligned.  The container
 * length is written into its header; read it with nz_container_bytes.
 * Reference: nvcomp ANSManager::configure_compression + compress,
 * cuda/high_level.cu:103-112. */
int nz_encode_exponents(const void *exp_in, uint64_t n, uint32_t lane_symbols,
                        void *container, uint64_t container_cap, void *scratch,
                        uint64_t scratch_bytes, void *stream);

/* Size in bytes of the scratch area built into the library (see below). */
uint64_t nz_static_scratch_bytes(void);

/* Same result as nz_encode_exponents, byte for byte, but the caller passes no
 * scratch and the call allocates nothing: no cudaMalloc, no cudaFree, no
 * allocating library routine.  It exists for hosts that may not allocate device
 * memory when they compress - a server whose arena already owns the whole GPU
 * and exposes no allocator to plugins, or a framework that forbids cudaMalloc /
 * cudaFree on its hot path because both synchronise the device.  The scratch is a
 * fixed 6 MiB array inside the library image; every GPU that loads the library
 * carries it until the process exits.
 *
 * Limit: nz_encode_scratch_bytes(n, lane_symbols) must not exceed
 * nz_static_scratch_bytes() (about 5.5 million symbols at lane_symbols 256, fewer
 * for short lane streams); larger requests return NZ_E_CAPACITY with a message
 * and leave the container untouched.
 *
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress) with that device current; make that first call outside
 * any stream capture.  All calls on a device share the one array, which keeps the
 * previous call's contents (the call clears what it needs zeroed itself): two
 * calls whose work overlaps on the GPU - different streams, or threads - race on
 * it and corrupt each other's output.  Serialise them, or use nz_encode_exponents.
 *
 * This entry point has no counterpart in the reference. */
int nz_encode_exponents_static_scratch(const void *exp_in, uint64_t n,
                                       uint32_t lane_symbols, void *container,
                                       uint64_t container_cap, void *stream);

/* Copies the container header to the host and returns the container length
 * in *total_bytes and the largest coded unit (16-bit words) in
 * *max_unit_words.  Synchronises the stream (the one host sync of a write).
 * Reference: nvcomp get_compressed_output_size, cuda/high_level.cu:114-115. */
int nz_container_bytes(const void *container, uint64_t *total_bytes,
                       uint32_t *max_unit_words, void *stream);

/* The same without the synchronisation: enqueues the copy of the 64-byte header
 * into `host_header64` (pinned host memory, 8-byte aligned) on the stream and
 * returns; once the stream has passed that point (an event the caller
 * records), nz_parse_header reads length and largest unit from the copy.  This
 * is how a write avoids stalling the host.  nz_parse_header is a host function
 * and returns NZ_E_FORMAT when the bytes are not a header.
 * Reference: none (the reference blocks, cuda/high_level.cu:114-115). */
int nz_container_header_async(const void *container, void *host_header64, void *stream);
int nz_parse_header(const void *host_header64, uint64_t *total_bytes, uint32_t *max_unit_words);

/* Decode the container into n exponent bytes.  `status` is a device u32 the
 * kernel ORs NZ_STATUS_* bits into (may be NULL).  max_unit_words is the
 * value nz_container_bytes returned (0 = assume the worst case).
 * Reference: nvcomp ANSManager::decompress, cuda/high_level.cu:184-192. */
int nz_decode_exponents(const void *container, uint64_t container_bytes,
                        uint64_t n, uint32_t lane_symbols,
                        uint32_t max_unit_words, void *exp_out, void *status,
                        void *stream);

/* ---- whole-tensor paths -------------------------------------------------- */

/* split + histogram + table + encode in one call: bf16[N] -> fractions +
 * container, byte for byte what nz_split_bf16 followed by nz_encode_exponents
 * give (with 9-bit probabilities at precision 7).  Two sweeps over the input: a
 * histogram of the exponent bytes, then a kernel that writes the fractions and
 * codes the exponents without storing them.  Buffers as for nz_split_bf16 /
 * nz_encode_exponents, scratch of nz_compress_scratch_bytes bytes.
 * Reference: Manager::_write_to_cache, cuda/high_level.cu:71-130. */
int nz_compress_bf16(const void *in_bf16, uint64_t n, int precision,
                     uint32_t lane_symbols, void *frac_out, void *container,
                     uint64_t container_cap, void *scratch,
                     uint64_t scratch_bytes, void *stream);

/* Decode the container and merge with the fractions straight into bf16[N];
 * the exponent bytes never travel through global memory.  No host sync.
 * Reference: Manager::_decompress_and_merge, cuda/high_level.cu:164-206. */
int nz_decompress_bf16(const void *container, uint64_t container_bytes,
                       const void *frac_in, uint64_t n, int precision,
                       uint32_t lane_symbols, uint32_t max_unit_words,
                       int canonical_nan, void *out_bf16, void *status,
                       void *stream);

/* Fused AdamW step on a decoded bf16 weight (in place): m and v are fp32 or
 * bf16 arrays of n elements (state_is_bf16), `step` counts from 1, the gradient
 * is multiplied by grad_scale first (1/world_size after a sum all-reduce).
 * w <- w*(1 - lr*wd) - lr/(1-b1^t) * m / (sqrt(v/(1-b2^t)) + eps), all in fp32,
 * rounded to bf16 once.  All four arrays 16-byte aligned.  It is the update
 * between the read and the write of the reference's in-backward step, which
 * uses plain SGD there.
 * Reference: compressed_lomo_hook, neuzip/__init__.py:25-35. */
int nz_adamw_bf16(void *weight_bf16, const void *grad_bf16, void *exp_avg,
                  void *exp_avg_sq, uint64_t n, int state_is_bf16, float lr,
                  float beta1, float beta2, float eps, float weight_decay,
                  uint32_t step, float grad_scale, void *stream);

/* The whole read -> update -> write cycle of one compressed weight in one call,
 * with the update fused into the decoder: the decode kernel applies the AdamW
 * step (the formula of nz_adamw_bf16, moments in bf16) to the weights as it
 * produces them, against the gradient and the moments at the same positions of
 * their row-major tensors, and writes the updated weights once, into `scratch`;
 * the compressor then codes them into frac_out / container_out (which may be
 * the buffers a previous call produced, but not the inputs of this one; read
 * the new container's size with nz_container_bytes).  operand_cols != 0 names
 * the row length of a weight stored in operand order (kept).  Results are bit
 * for bit those of nz_decompress_bf16 -> nz_adamw_bf16 -> nz_compress_bf16.
 * Scratch of nz_adamw_compressed_scratch_bytes bytes, 16-byte aligned.
 * Reference: compressed_lomo_hook (neuzip/__init__.py:25-35: param() ->
 * add_ -> manager.write) and the loop at examples/training/train_clm.py:822-833. */
uint64_t nz_adamw_compressed_scratch_bytes(uint64_t n, uint32_t lane_symbols);
int nz_adamw_compressed_bf16(const void *container, uint64_t container_bytes, const void *frac_in,
                             uint64_t n, uint64_t operand_cols, int precision,
                             uint32_t lane_symbols, uint32_t max_unit_words, int canonical_nan,
                             const void *grad_bf16, void *exp_avg_bf16, void *exp_avg_sq_bf16,
                             float lr, float beta1, float beta2, float eps, float weight_decay,
                             uint32_t step, float grad_scale, void *frac_out, void *container_out,
                             uint64_t container_cap, void *scratch, uint64_t scratch_bytes,
                             void *status, void *stream);

/* Item flag: the container and the fractions were complete (written and
 * visible) before the kernel that precedes this call on the stream was
 * launched -- true for weights that were compressed earlier and are decoded
 * again and again.  When every item of a launch says so, the launch builds its
 * decode table while the previous kernel drains instead of after it.  Never
 * set it for data written by the work enqueued just before the call. */
#define NZ_ITEM_INPUTS_STABLE 0x1u

/* One tensor of a batched decompress. */
typedef struct nz_decompress_item {
  const void *container;     /* NZR1 container, 16-byte aligned            */
  uint64_t container_bytes;
  const void *frac_in;       /* packed fractions, 8-byte aligned           */
  uint64_t n;                /* elements                                   */
  uint32_t max_unit_words;   /* from nz_container_bytes, 0 = worst case    */
  uint32_t flags;            /* NZ_ITEM_* bits, 0 = none                   */
  void *out_bf16;            /* bf16[n], 16-byte aligned                   */
  uint64_t operand_cols;     /* 0, or the row length of a matrix stored in
                                operand order (nz_compress_bf16_operand);
                                the output is row-major either way          */
  uint32_t lane_symbols;     /* 0 = the call's lane_symbols; else this
                                tensor's own (tensors of one call may differ) */
  uint32_t normalizer_group; /* group size of the block normaliser, when
                                `normalizers` is set (a power of two <= 1024) */
  const void *normalizers;   /* NULL, or the bytes nz_normalize_bf16 wrote:
                                the decoder multiplies every group by its
                                scale as it writes it (stream order only),
                                which replaces nz_denormalize_bf16          */
} nz_decompress_item;

/* nz_decompress_bf16 for several tensors of the same precision (for instance the
 * seven matrices of one transformer layer; an item may name its own lane_symbols) in
 * as few launches as possible: up to 8 tensors share a launch, each on a share
 * of the SMs proportional to its size, so small matrices do not leave most of
 * the GPU idle and the fixed cost of a launch is paid once.  `items` is a host
 * array; results are the same as `count` single calls.  No host sync.
 * Reference: Manager::read called once per converted Linear while a layer runs
 * (neuzip/nn/module.py:23-25 -> neuzip/binding.py:88-92 -> cuda/high_level.cu:223-250). */
int nz_decompress_bf16_batch(const nz_decompress_item *items, uint32_t count,
                             int precision, uint32_t lane_symbols,
                             int canonical_nan, void *status, void *stream);

/* Gather: decode only the units named in `unit_ids` (a device array of n_ids
 * unit numbers, each < ceil(n / (32 * lane_symbols)); a unit is 32 *
 * lane_symbols consecutive elements) and write them one after the other:
 * unit_ids[i] goes to out_bf16[i * 32 * lane_symbols ...], which must hold
 * n_ids units (the tensor's last unit may be shorter; only its elements are
 * written).  A number may appear more than once.  Numbers out of range set
 * NZ_STATUS_BAD_UNIT and write nothing.  The container is the one
 * nz_compress_bf16 wrote: units are independently decodable by construction.
 * Reference: Embedding.forward decompresses the whole table for every lookup
 * (neuzip/nn/embedding.py:30-39 -> cuda/high_level.cu:223-250); with this call
 * a lookup decodes the rows it touches. */
int nz_decompress_bf16_units(const void *container, uint64_t container_bytes,
                             const void *frac_in, uint64_t n, int precision,
                             uint32_t lane_symbols, uint32_t max_unit_words,
                             int canonical_nan, const void *unit_ids, uint32_t n_ids,
                             void *out_bf16, void *status, void *stream);

/* Row gather on top of nz_decompress_bf16_units: the tensor is a table of
 * n / row_len rows; row rows_i64[i] (a device array of n_rows_out int64) is
 * written to out_bf16[i * row_len ...].  Three launches, no host sync: the unit
 * list is built on the device, those units are decoded into `scratch`
 * (nz_gather_scratch_bytes; 16-byte aligned), the rows are copied out.  Row
 * numbers outside the table set NZ_STATUS_BAD_UNIT and leave their output row
 * untouched.  Reference: Embedding.forward = F.embedding(x, whole decompressed
 * table) (neuzip/nn/embedding.py:30-39). */
uint64_t nz_gather_scratch_bytes(uint32_t n_rows_out, uint64_t row_len, uint32_t lane_symbols);
int nz_gather_rows_bf16(const void *container, uint64_t container_bytes,
                        const void *frac_in, uint64_t n, int precision,
                        uint32_t lane_symbols, uint32_t max_unit_words,
                        int canonical_nan, uint64_t row_len, const void *rows_i64,
                        uint32_t n_rows_out, void *out_bf16, void *scratch,
                        uint64_t scratch_bytes, void *status, void *stream);

/* nz_gather_rows_bf16 for a table written with a block normaliser: the rows come
 * out multiplied by their groups' scales (normalizers = the bytes
 * nz_normalize_bf16 wrote for the whole table, normalizer_group its group size;
 * NULL / 0 = none).
 * Reference: cuda/kernels.cuh:208-216 inside Embedding.forward's full read. */
int nz_gather_rows_normalized_bf16(const void *container, uint64_t container_bytes,
                                   const void *frac_in, uint64_t n, int precision,
                                   uint32_t lane_symbols, uint32_t max_unit_words,
                                   int canonical_nan, uint64_t row_len, const void *rows_i64,
                                   uint32_t n_rows_out, const void *normalizers,
                                   uint32_t normalizer_group, void *out_bf16, void *scratch,
                                   uint64_t scratch_bytes, void *status, void *stream);

/* y = W x (+ bias) for one input vector, with W the compressed [out, in]
 * row-major bf16 matrix of n = out * in elements: the weights are multiplied as
 * they are decoded and never written back.  in_features must be a multiple of
 * 256.  x_f32 is the input vector in fp32 (in entries, 16-byte aligned), bias
 * (bf16, out entries) may be NULL, y_bf16 receives out bf16 values (products
 * and sums in fp32, one rounding at the end).  Two launches, no host sync:
 * the decode kernel leaves per-unit partial sums in `scratch`
 * (nz_linear_vec_scratch_bytes, 16-byte aligned), a second kernel adds them
 * per row in a fixed order, so the result is reproducible run to run.
 * Reference: Manager::linear / linear_without_bias = full decompress, then a
 * library GEMM (cuda/high_level.cu:252-263; neuzip/nn/module.py:27-28). */
uint64_t nz_linear_vec_scratch_bytes(uint64_t n, uint64_t in_features, uint32_t lane_symbols);
int nz_linear_vec_bf16(const void *container, uint64_t container_bytes,
                       const void *frac_in, uint64_t n, int precision,
                       uint32_t lane_symbols, uint32_t max_unit_words,
                       int canonical_nan, uint64_t in_features, const void *x_f32,
                       const void *bias_bf16, void *y_bf16, void *scratch,
                       uint64_t scratch_bytes, void *status, void *stream);

/* ---- operand order and the fused linear ----------------------------------- */

/* A [rows, cols] weight matrix can be stored in "operand order": the codec is
 * applied to a permutation of the matrix in which every 256-element block of
 * the stream is a 4-row x 64-column patch (stream element
 * ((g * cols/64 + kb) * 4 + r) * 64 + c  is matrix element (4g + r, 64kb + c)),
 * so that what the decoder produces per step is a piece of a tensor-core
 * operand tile.  Requirements: rows % 4 == 0, cols % 64 == 0 and lane_symbols / 8
 * divides cols / 64 (a unit never straddles a row group).  The stored bytes are
 * what nz_compress_bf16 produces for the permuted tensor; the reference never
 * exposes its stored bytes (cuda/high_level.cu:35-43), only what write / read
 * return, which is unchanged. */

/* lane_symbols to use for a matrix with `cols` columns at `precision`: the
 * admissible value closest to nz_default_lane_symbols, or 0 when the matrix
 * cannot be stored in operand order. */
uint32_t nz_operand_lane_symbols(uint64_t cols, int precision);

/* The same for a matrix whose row count is known: the unit length (16 to 48
 * blocks of 64 columns) with which nz_linear_bf16 has the fewest decode steps in
 * sequence on the 148 SMs of a B200 - one work item per 128-row tile and
 * unit-long column segment, run in waves of 148.  Falls back to the rule above
 * when cols / 64 has no divisor in that range; rows = 0 means "unknown". */
uint32_t nz_operand_lane_symbols_for(uint64_t rows, uint64_t cols, int precision);

/* nz_compress_bf16 for a row-major [rows, cols] matrix, stored in operand order.
 * Scratch of nz_compress_operand_scratch_bytes bytes.
 * Reference: Manager::_write_to_cache, cuda/high_level.cu:71-130. */
uint64_t nz_compress_operand_scratch_bytes(uint64_t rows, uint64_t cols, uint32_t lane_symbols);
int nz_compress_bf16_operand(const void *in_bf16, uint64_t rows, uint64_t cols, int precision,
                             uint32_t lane_symbols, void *frac_out, void *container,
                             uint64_t container_cap, void *scratch, uint64_t scratch_bytes,
                             void *stream);

/* nz_decompress_bf16 for a matrix stored in operand order; out_bf16 receives the
 * row-major [rows, cols] matrix.
 * Reference: Manager::_decompress_and_merge, cuda/high_level.cu:164-206. */
int nz_decompress_bf16_operand(const void *container, uint64_t container_bytes,
                               const void *frac_in, uint64_t rows, uint64_t cols, int precision,
                               uint32_t lane_symbols, uint32_t max_unit_words, int canonical_nan,
                               void *out_bf16, void *status, void *stream);

/* y[m_tokens, rows] = x[m_tokens, cols] * W^T (+ bias) for a weight W[rows, cols]
 * stored in operand order: the decoder writes the bf16 weight tiles into shared
 * memory in the tensor cores' operand layout and tcgen05.mma consumes them there
 * (fp32 accumulation in tensor memory, one rounding to bf16 at the end), so the
 * decoded weight never travels through global memory.  x and y are row-major
 * bf16 (x 16-byte aligned), bias is bf16[rows] or NULL.  When a row of W spans
 * several units (cols / 64 > lane_symbols / 8) each column segment is summed on
 * its own into `workspace` (nz_linear_workspace_bytes, 16-byte aligned, fp32) and
 * a second kernel adds the segments in a fixed order, so results are
 * reproducible run to run.  Inputs of more than 256 rows are processed 256 at a
 * time, decoding the weight once per pass.  No host sync.  Faults found while
 * decoding are reported in `status` as for nz_decompress_bf16.
 * Reference: Manager::linear / linear_without_bias = full decompress into a new
 * tensor, then a library GEMM (cuda/high_level.cu:252-263). */
uint64_t nz_linear_workspace_bytes(uint64_t rows, uint64_t cols, uint32_t lane_symbols,
                                   uint64_t m_tokens);
int nz_linear_bf16(const void *container, uint64_t container_bytes, const void *frac_in,
                   uint64_t rows, uint64_t cols, int precision, uint32_t lane_symbols,
                   uint32_t max_unit_words, int canonical_nan, const void *x_bf16,
                   uint64_t m_tokens, const void *bias_bf16, void *y_bf16, void *workspace,
                   uint64_t workspace_bytes, void *status, void *stream);

/* ---- the fused linear with a tensor-parallel all-reduce in its epilogue ------ */

/* Row-parallel Linears of a tensor-parallel model (each rank holds a block of
 * input columns) produce partial sums that have to be added over the ranks.
 * nz_linear_allreduce_bf16 is nz_linear_bf16 with that all-reduce fused in: the
 * kernel's epilogue writes its fp32 sums straight from tensor memory into EVERY
 * rank's workspace with plain peer stores over NVLink (plane [source rank][row of
 * x][row of W]; when the shard has several column segments, the CTAs of a row
 * tile first add their partial sums locally, in segment order, and the last one
 * to arrive does the peer stores), fences at system scope and adds one arrival
 * per CTA to every rank's arrival counters; a second kernel on each rank waits
 * (bounded: about a second, then NZ_STATUS_TIMEOUT) until every rank's CTAs of
 * the call have arrived and adds the planes rank by rank, so every rank obtains
 * the same bits.  No multicast, no library collective.  All ranks must make the same sequence of calls (same shapes);
 * arrival counters only grow: pass the value *arrivals_after of the previous
 * call on the same buffers as arrivals_before (0 at first).  A buffer set may be
 * reused by the call after next at the earliest, so alternate two sets.  The
 * bias, if any, is given on ONE rank only (it joins that rank's partial sums).
 * Reference: none - the reference has no tensor parallelism; the baseline is
 * nz_linear_bf16 followed by an NCCL all-reduce. */
typedef struct nz_peer_group {
  uint32_t world, rank;       /* 2..8 ranks, this rank's number                */
  void *workspace[8];         /* every rank's workspace as seen from this GPU  */
  void *arrivals[8];          /* every rank's u32[8] arrival counters          */
  uint64_t workspace_bytes;   /* size of each workspace                        */
} nz_peer_group;

uint64_t nz_linear_allreduce_workspace_bytes(uint64_t rows, uint64_t cols, uint32_t lane_symbols,
                                             uint64_t m_tokens, uint32_t world);
int nz_linear_allreduce_bf16(const void *container, uint64_t container_bytes, const void *frac_in,
                             uint64_t rows, uint64_t cols, int precision, uint32_t lane_symbols,
                             uint32_t max_unit_words, int canonical_nan, const void *x_bf16,
                             uint64_t m_tokens, const void *bias_bf16, void *y_bf16,
                             const nz_peer_group *peers, uint32_t arrivals_before,
                             uint32_t *arrivals_after, void *status, void *stream);

/* Peer-visible device memory for the call above (these four allocate or map
 * memory and synchronise; call them at set-up).  nz_peer_alloc: cudaMalloc,
 * zero, and export a 64-byte inter-process handle; nz_peer_open: map a peer's
 * handle into this process (peer access is enabled on demand).
 * Reference: none. */
int nz_peer_alloc(uint64_t bytes, void **ptr, void *handle64);
int nz_peer_open(const void *handle64, void **ptr);
int nz_peer_close(void *ptr);
int nz_peer_free(void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* NEUZIP_B200_H_ */
