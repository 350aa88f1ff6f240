/*
 * b200ew -- C ABI of the B200 compound-optree runtime (libb200ew.so).
 *
 * This library is what the Python backend binds with ctypes.  It takes the
 * place of the pycuda driver bindings that neon's NervanaGPU backend uses on
 * the op-tree path; each group below names the reference call sites it
 * replaces (paths are relative to the neon source tree).
 *
 * Conventions
 *   - every function returns a b200_status (0 = OK, negative = error class);
 *     nothing throws, nothing aborts.  b200_last_error() returns the message
 *     of the calling thread's last failure.  (neon's own C API returns bool:
 *     neon/backends/kernels/C_interface/nervana_c_api.h:31-105.)
 *   - device pointers, streams, events, kernels and communicators travel as
 *     uint64_t handles; 0 is the null handle (stream 0 = the library's stream
 *     of the current device).
 *   - one process drives one device: b200_init(dev) selects it for the calling
 *     process.  Calls are thread-compatible, not thread-safe.
 *   - host buffers are borrowed for the duration of the call.
 */
#ifndef B200EW_H
#define B200EW_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t b200_status;

#define B200_OK               0
#define B200_ERR_INVALID     -1   /* bad argument / bad handle            */
#define B200_ERR_CUDA        -2   /* CUDA runtime call failed             */
#define B200_ERR_COMPILE     -3   /* NVRTC rejected the kernel source     */
#define B200_ERR_OOM         -4   /* device or pinned memory exhausted    */
#define B200_ERR_NCCL        -5   /* NCCL missing or a collective failed  */
#define B200_ERR_TIMEOUT     -6   /* a bounded device-side wait gave up   */
#define B200_ERR_UNSUPPORTED -7

/* element types of tensors (numpy dtype.str[1:] in the reference:
 * neon/backends/cuda_templates.py:386-435) */
#define B200_F32 0
#define B200_F16 1
#define B200_BF16 2
#define B200_I32 3
#define B200_U32 4
#define B200_I16 5
#define B200_U16 6
#define B200_I8  7
#define B200_U8  8

/* reduction operators (neon/backends/cuda_templates.py:577-613) */
#define B200_SUM 0
#define B200_MAX 1
#define B200_MIN 2

typedef struct b200_device_props {
    int32_t sm_count;
    int32_t cc_major, cc_minor;
    int32_t max_smem_per_block;      /* opt-in dynamic shared memory, bytes */
    int32_t max_threads_per_sm;
    int32_t l2_bytes;
    int32_t clock_khz;
    int32_t reserved;
    uint64_t total_mem;
    char name[64];
} b200_device_props;

/* ---- library / error ----------------------------------------------------- */
int32_t     b200_version(void);
size_t      b200_last_error(char *buf, size_t n);      /* returns message length */

/* ---- device and context
 * replaces drv.init / Device(id).make_context / ctx.detach
 * (neon/backends/nervanagpu.py:717-811, util/check_gpu.py) */
b200_status b200_device_count(int32_t *count);
b200_status b200_init(int32_t device);
b200_status b200_shutdown(void);
b200_status b200_device_props_get(int32_t device, b200_device_props *out);
b200_status b200_mem_info(uint64_t *free_bytes, uint64_t *total_bytes);

/* ---- device memory: caching arena, 256-byte aligned blocks
 * replaces drv.mem_alloc as GPUTensor's allocator, the shape-keyed temp pool
 * and the scratch buffer (neon/backends/nervanagpu.py:87,147,836-890,1051-1075) */
b200_status b200_malloc(uint64_t bytes, uint64_t *dptr);
b200_status b200_free(uint64_t dptr);                   /* reuse is ordered by the library's stream; while streams made
                                                           with b200_stream_create exist, the block is reused only after
                                                           the work queued on every stream at this moment has run */
b200_status b200_mem_trim(void);                        /* give cached blocks back */
b200_status b200_mem_stats(uint64_t *in_use, uint64_t *cached, uint64_t *peak_in_use,
                           uint64_t *device_allocs);
b200_status b200_host_alloc(uint64_t bytes, void **hptr);   /* pinned */
b200_status b200_host_free(void *hptr);

/* ---- copies and fills
 * replaces drv.memcpy_htod_async / memcpy_dtoh_async / memcpy_dtod_async and
 * memset_d8/d16/d32_async (neon/backends/nervanagpu.py:350-369,385-435) */
b200_status b200_memcpy_h2d(uint64_t dst, const void *src, uint64_t bytes, uint64_t stream, int32_t sync);
b200_status b200_memcpy_d2h(void *dst, uint64_t src, uint64_t bytes, uint64_t stream, int32_t sync);
b200_status b200_memcpy_d2d(uint64_t dst, uint64_t src, uint64_t bytes, uint64_t stream);
b200_status b200_memset(uint64_t dst, uint32_t value, int32_t width, uint64_t count, uint64_t stream);

/* ---- streams and events
 * replaces be.stream and the timing marks init_mark / record_mark /
 * synchronize_mark / get_time (neon/backends/nervanagpu.py:780,3138-3177,3279-3281) */
b200_status b200_stream_create(uint64_t *stream);
b200_status b200_stream_destroy(uint64_t stream);
b200_status b200_stream_sync(uint64_t stream);
b200_status b200_stream_wait_event(uint64_t stream, uint64_t event);
b200_status b200_default_stream(uint64_t *stream);
b200_status b200_event_create(uint64_t *event);
b200_status b200_event_destroy(uint64_t event);
b200_status b200_event_record(uint64_t event, uint64_t stream);
b200_status b200_event_sync(uint64_t event);
b200_status b200_event_elapsed_ms(uint64_t start, uint64_t end, float *ms);

/* ---- kernels: NVRTC instantiation of op-tree signatures, cached
 * replaces pycuda SourceModule(code) + get_function + prepare
 * (neon/backends/float_ew.py:268,611-615; disk cache: util/source_module.py:11-22).
 * b200_register_header makes an in-memory header available to #include. */
b200_status b200_register_header(const char *name, const char *source);
b200_status b200_nvrtc_compile(const char *source, const char *const *options, int32_t n_options,
                               void **image, uint64_t *image_size, int32_t *from_cache);
b200_status b200_buffer_free(void *image);
b200_status b200_kernel_get(const char *source, const char *kernel_name,
                            const char *const *options, int32_t n_options, uint64_t *kernel);
b200_status b200_kernel_max_smem(uint64_t kernel, int32_t bytes);
b200_status b200_kernel_occupancy(uint64_t kernel, int32_t block_threads, int32_t smem_bytes,
                                  int32_t *blocks_per_sm);
b200_status b200_kernel_max_clusters(uint64_t kernel, int32_t block_threads, int32_t smem_bytes,
                                     int32_t cluster_size, int32_t grid_blocks, int32_t *clusters);
b200_status b200_cache_stats(uint64_t *compiled, uint64_t *disk_hits, uint64_t *memory_hits);

/* ---- launch
 * replaces kernel.prepared_async_call(grid, block, stream, *args, shared_size)
 * (neon/backends/float_ew.py:929-931).  `params` is the kernel's single
 * by-value parameter struct (<= 4096 bytes).  cluster_x > 1 launches
 * thread-block clusters.  `cooperative` is a set of bits: 1 guarantees
 * co-residency of the grid; 2 says that the kernel executes griddepcontrol.wait
 * before its first memory access, so its blocks may be scheduled while the
 * previous kernel of the stream drains (programmatic dependent launch). */
b200_status b200_launch(uint64_t kernel, uint32_t grid_x, uint32_t grid_y, uint32_t grid_z,
                        uint32_t block_x, uint32_t block_y, uint32_t block_z,
                        uint32_t smem_bytes, uint64_t stream,
                        const void *params, uint32_t params_size,
                        uint32_t cluster_x, int32_t cooperative);

/* ---- CUDA graphs: record the launches of a statement sequence once, replay them with one call
 * no counterpart in the reference (it predates CUDA graphs); answers the same problem its
 * memoised stacks do (neon/backends/nervanagpu.py:662-691): per-statement host work that is
 * larger than the kernels for small tensors.  Between begin and end every launch / fill / device
 * copy on `stream` is recorded instead of run; allocation, compilation and host transfers are not
 * allowed there (run the sequence once eagerly first).  Pointers and numbers are frozen as
 * recorded. */
b200_status b200_graph_begin(uint64_t stream);
b200_status b200_graph_end(uint64_t stream, uint64_t *graph_exec);
b200_status b200_graph_launch(uint64_t graph_exec, uint64_t stream);
b200_status b200_graph_destroy(uint64_t graph_exec);

/* ---- random state: counter-based generator keyed by (seed, launch number)
 * replaces the 3x65536-word LFSR pool and gen_rng / rng_reset / rng_get_state /
 * rng_set_state (neon/backends/nervanagpu.py:901-1049, cuda_templates.py:138-186) */
b200_status b200_rng_seed(uint64_t seed);
b200_status b200_rng_next_key(uint32_t key[2]);       /* advances the launch counter */
b200_status b200_rng_get_state(uint64_t state[2]);    /* {seed, launch counter} */
b200_status b200_rng_set_state(const uint64_t state[2]);

/* ---- whole-tensor reduction with fixed kernels (no run-time compilation)
 * the axis=None case of be.sum / be.max / be.min (neon/backends/backend.py:1313-1380),
 * which the reference runs as two launches through a pooled temporary
 * (neon/backends/nervanagpu.py:1158-1170).  `scratch` is caller-provided device
 * memory of at least b200_reduce_scratch_bytes() bytes; its first 8 bytes must be
 * zero before the first use and are left zero by every call.  The fp32 result
 * is written to `out`.  absolute != 0 reduces |x|. */
uint64_t    b200_reduce_scratch_bytes(void);
b200_status b200_reduce_full(uint64_t in, int32_t dtype, uint64_t count, int32_t op, int32_t absolute,
                             uint64_t out, uint64_t scratch, uint64_t stream);

/* ---- matrix product for `dot` nodes inside op-trees
 * stands in for compound_dot on the op-tree path only (neon/backends/nervanagpu.py:1123-1146,
 * 1275-1281, 1441-1622): C = alpha * A.B + beta * C with element strides (so transposed views
 * work), f32/f16 operands, fp32 accumulation.  A plain shared-memory tiled kernel: it is there
 * so that trees containing dot evaluate, not to compete with the SASS GEMMs of the reference. */
b200_status b200_gemm(uint64_t a, int32_t a_dtype, int64_t a_stride0, int64_t a_stride1,
                      uint64_t b, int32_t b_dtype, int64_t b_stride0, int64_t b_stride1,
                      uint64_t c, int32_t c_dtype, int64_t c_stride0, int64_t c_stride1,
                      int32_t m, int32_t n, int32_t k, float alpha, float beta, uint64_t stream);

/* ---- dimension shuffle (copy with permuted axes)
 * replaces copy_transpose (neon/backends/nervanagpu.py:3077-3118; kernel generator
 * _get_copy_transpose_kernel in neon/backends/convolution.py), which the data iterator
 * calls once per minibatch to turn (examples, features) rows into neon's (features, batch)
 * layout (neon/data/dataiterator.py:144-202).  The copy is described in OUTPUT dimension
 * order: shape[i] is the extent of output dimension i, dst_strides[i] the output's element
 * stride there and src_strides[i] the element stride of the input axis that lands there
 * (a.strides[axes[i]]).  Views are fine (any non-negative strides); the two tensors must
 * not overlap.  elem_bytes in {1,2,4,8}; at most B200_SHUFFLE_MAX_DIMS dimensions. */
#define B200_SHUFFLE_MAX_DIMS 8
b200_status b200_dimshuffle(uint64_t dst, uint64_t src, int32_t elem_bytes, int32_t ndim,
                            const int64_t *shape, const int64_t *dst_strides,
                            const int64_t *src_strides, uint64_t stream);

/* ---- Kahan-compensated accumulation
 * replaces NervanaGPU.compensated_sum (neon/backends/nervanagpu.py:1896-1917; kernel text
 * neon/backends/float_ew.py:944-1037): sum += add*add_scale - cmp*cmp_scale with the
 * rounding error of the stored sum kept in cmp.  sum, cmp and add are contiguous arrays of
 * `count` elements of one dtype (f32, f16, bf16).  rounding_bits > 0 rounds the new sum
 * stochastically to that many mantissa bits (capped at 15 / 10 / 7) with the library's
 * seeded generator, and advances its launch counter; 0 rounds to nearest. */
b200_status b200_compensated_sum(uint64_t sum, uint64_t cmp, uint64_t add, int32_t dtype, uint64_t count,
                                 float cmp_scale, float add_scale, int32_t rounding_bits, uint64_t stream);

/* ---- histogram of binary orders of magnitude
 * replaces GPUTensor.hist -> _compute_hist (neon/backends/nervanagpu.py:619-637,
 * neon/backends/float_ew.py:1069-1158): hist[b] = number of elements with
 * clamp(round(log2|x|) - offset, 0, nbins - 1) == b, for a contiguous array of any supported
 * dtype (integers are binned by their value converted to float).
 * `hist` (nbins int32 counters) is zeroed by the call.  nbins <= B200_HIST_MAX_BINS. */
#define B200_HIST_MAX_BINS 128
b200_status b200_log2_hist(uint64_t in, int32_t dtype, uint64_t count, uint64_t hist, int32_t nbins,
                           int32_t offset, uint64_t stream);

/* ---- the same reduction for callers that cannot allocate device memory
 * No counterpart in the reference.  Meant for hosts where cudaMalloc is off
 * limits when the call is made (a framework pool owns the device, a latency-
 * critical loop, memory already handed out): the split-reduction scratch is a
 * fixed 16640-byte array inside the library image, resident on every GPU that
 * loads the library until the process exits.  The call allocates nothing and
 * takes no scratch argument; inputs and the 4-byte fp32 output are the
 * caller's.  Limits and rules:
 *   - count <= B200_NOALLOC_MAX_COUNT, larger inputs are refused with
 *     B200_ERR_INVALID (use b200_reduce_full with your own scratch);
 *   - the first call on a device looks up the array's device address (the
 *     device must be current); make that call before starting a stream capture;
 *   - all calls on a device share the one array: calls that can overlap on the
 *     GPU (different streams, no ordering between them) race and give wrong
 *     results; order them on one stream or with events;
 *   - stream 0 means the library's stream after b200_init, else the default stream. */
#define B200_NOALLOC_MAX_COUNT (1ull << 32)
uint64_t    b200_reduce_full_noalloc_max_count(void);
b200_status b200_reduce_full_noalloc(uint64_t in, int32_t dtype, uint64_t count, int32_t op, int32_t absolute,
                                     uint64_t out, uint64_t stream);

/* ---- collectives over NVLink (NCCL, loaded at run time)
 * no counterpart in the reference tree: its multi-GPU backend was a closed
 * package (neon/backends/__init__.py:42-46).  Used to finish reductions that
 * cross the sharded (batch/column) axis. */
b200_status b200_comm_unique_id(uint8_t id[128]);
b200_status b200_comm_init(const uint8_t id[128], int32_t n_ranks, int32_t rank, uint64_t *comm);
b200_status b200_comm_destroy(uint64_t comm);
b200_status b200_allreduce(uint64_t comm, uint64_t send, uint64_t recv, uint64_t count,
                           int32_t dtype, int32_t op, uint64_t stream);
b200_status b200_allgather(uint64_t comm, uint64_t send, uint64_t recv, uint64_t send_bytes,
                           uint64_t stream);

/* ---- exchange areas: peer-mapped device memory for reductions that finish across GPUs
 * inside the reduction kernel (no counterpart in the reference tree, as above).  Collective
 * over `comm`: every rank allocates `bytes` (zeroed) on its device, the CUDA IPC handles
 * travel over the communicator, every rank maps the others' areas.  *local is this rank's
 * area; *table is a device array of n_ranks addresses, entry r = rank r's area as this device
 * addresses it.  Kernels write partial results and a launch number into the peers' areas with
 * plain stores over NVLink and read only their own area; they never wait without a time limit. */
b200_status b200_xchg_create(uint64_t comm, int32_t n_ranks, int32_t rank, uint64_t bytes,
                             uint64_t *local, uint64_t *table);
b200_status b200_xchg_destroy(uint64_t local);

#ifdef __cplusplus
}
#endif
#endif /* B200EW_H */
