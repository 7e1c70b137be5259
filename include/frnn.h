/*
 * frnn.h - C ABI of libfrnn_b200.so, the launch boundary of the B200 backend
 * for flex_rnn step functions.
 *
 * In the reference project the generated CUDA is wrapped, per compiled step,
 * in host stubs `void <kernel>_(void* ...)` that launch with a baked
 * `<<<grid, block>>>` on the legacy default stream, and those stubs are bound
 * as torch ops taking tensors and passing `data_ptr()`
 * (flex_rnn/to_cuda.py:230-280: `build_cuda`).  This library is what replaces
 * that boundary: the generated source is compiled at run time with NVRTC for
 * sm_100a and launched on a caller-supplied stream through the functions
 * below.  Plain pointers and sizes only; no torch types cross this boundary.
 *
 * Conventions: every function returns 0 on success and a non-zero FRNN_E_*
 * code on failure; nothing throws; `frnn_last_error()` gives a per-thread
 * message for the last failure.  The caller owns every device buffer; kernels
 * only read their inputs and write the buffers passed as outputs.  All calls
 * are thread-safe.  A module belongs to the device that was current when it
 * was loaded.
 */
#ifndef FRNN_H
#define FRNN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    FRNN_OK = 0,
    FRNN_E_ARG = 1,        /* bad argument */
    FRNN_E_NVRTC = 2,      /* NVRTC missing or compilation failed (see log) */
    FRNN_E_DRIVER = 3,     /* CUDA driver missing or a driver call failed */
    FRNN_E_LAUNCH = 4,     /* launch rejected (resources, configuration) */
    FRNN_E_KERNEL = 5      /* a kernel reported an error through its error word */
};

typedef struct frnn_module* frnn_module_t;

/* Version of this ABI (bumped on any signature change). */
int frnn_abi_version(void);

/* Message for the calling thread's most recent failure ("" if none). */
const char* frnn_last_error(void);

/* Version of the NVRTC that frnn_compile uses (12, 8 for NVRTC 12.8).  A cubin
 * cache must key on it: the reference keys its build directory on the source
 * hash alone (flex_rnn/to_cuda.py:264) and relies on ninja to rebuild. */
int frnn_nvrtc_version(int* major, int* minor);

/*
 * Compile CUDA C++ `src` to an sm_100a cubin with NVRTC (no GPU needed).
 * Replaces the nvcc+ninja build of flex_rnn/to_cuda.py:274-279.
 * `opts`: extra NVRTC options (may be NULL when nopts == 0).
 * On success *cubin is a malloc'd buffer of *cubin_size bytes that the caller
 * releases with frnn_free().  `log` (may be NULL) receives the NUL-terminated
 * compiler log, truncated to log_cap bytes; it holds the ptxas resource usage
 * (registers, spills, shared memory) of every kernel.
 */
int frnn_compile(const char* src, const char* const* opts, int nopts,
                 void** cubin, size_t* cubin_size, char* log, size_t log_cap);

void frnn_free(void* p);

/*
 * Load a cubin on the current device and look up `nkernels` entry points by
 * name.  Replaces the dlopen of the extension built by to_cuda.py:279-280.
 * Raises each kernel's dynamic shared memory limit to `smem_bytes[i]`.
 */
int frnn_module_load(const void* cubin, size_t cubin_size,
                     const char* const* kernel_names, const unsigned* smem_bytes,
                     int nkernels, frnn_module_t* out);

int frnn_module_unload(frnn_module_t m);

/*
 * Launch kernel `kernel` of module `m` on `stream` (a cudaStream_t / CUstream;
 * NULL = default stream).  `args[i]` points at the i-th kernel parameter value
 * (for a pointer parameter: the address of a variable holding the device
 * pointer), as for cuLaunchKernel.  Replaces the `<<<grid, block>>>` stubs of
 * flex_rnn/to_cuda.py:245-247, adding the stream argument and error checking
 * that those stubs lack.  Asynchronous: returns once the launch is enqueued.
 */
int frnn_launch(frnn_module_t m, int kernel, const unsigned grid[3], const unsigned block[3],
                unsigned smem_bytes, void* stream, void* const* args, int nargs);

/*
 * Encode a TMA tensor map (a 128-byte opaque descriptor, 64-byte aligned, in
 * host memory at `out_map`) for a tiled `cp.async.bulk.tensor` load from the
 * tensor at device address `base`: `rank` dimensions (1..5, fastest first) of
 * `dims[i]` elements of `elt_bytes` bytes, byte strides `strides_bytes[i]` for
 * dimensions 1..rank-1 (multiples of 16), and a box of `box[i]` elements.
 * The generated kernels take such maps as `__grid_constant__` parameters: pass
 * the address of the 128 bytes as that parameter's entry of `args`.  (No
 * counterpart in the reference, whose kernels use scalar global loads,
 * to_cuda.py:148-170.)  Out-of-range parts of a box read as zero.
 */
int frnn_tensor_map_encode(void* out_map, const void* base, unsigned elt_bytes, unsigned rank,
                           const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box);

/*
 * Kernel error word.  Every device-side wait of the generated kernels is
 * time-bounded; a kernel whose wait ran out writes a non-zero code into the
 * `int` error word it was given as its last pointer parameter and returns
 * early, so its outputs are not valid.  A kernel compiled with -DFRNN_BOUNDS
 * (the checked build: every access is tested against the byte extents the
 * generator registered for the kernel's buffers) writes code 64 when it
 * refused an access outside them.  (The reference has no counterpart: its
 * stubs check nothing, flex_rnn/to_cuda.py:245-252.)  The word is sticky until
 * one of the calls below clears it.  It may live in device memory or in pinned
 * host memory, which the device writes directly under unified addressing; the
 * Python host side uses the latter and calls frnn_status_check(word, NULL, NULL)
 * before each launch, which needs neither a copy nor a wait.
 *
 * frnn_status:       copies the word to the host on `stream`, waits for the
 *                    stream, and returns FRNN_E_KERNEL (word cleared, message
 *                    in frnn_last_error) if it was non-zero.  Synchronises.
 * frnn_status_post:  enqueues the copy of the word into `host_word` (pinned
 *                    host memory for a truly asynchronous copy) behind the
 *                    launches already on `stream`.  Does not wait.
 * frnn_status_check: looks at `host_word` as it is now, without waiting: 0 ->
 *                    FRNN_OK; otherwise clears `host_word`, enqueues a clear of
 *                    `err_word_dev` (may be NULL) on `stream` and returns
 *                    FRNN_E_KERNEL.  Called at the start of the next operation
 *                    it reports what the previous launches left, at no cost on
 *                    the hot path.
 */
int frnn_status(int* err_word_dev, void* stream);
int frnn_status_post(int* err_word_dev, int* host_word, void* stream);
int frnn_status_check(int* host_word, int* err_word_dev, void* stream);

/* Registers per thread, static shared bytes and local (spill) bytes per thread
 * of a loaded kernel, as the driver reports them. */
int frnn_kernel_attrs(frnn_module_t m, int kernel, int* regs, int* static_smem, int* local_bytes);

/*
 * frnn_launch for callers that must not allocate device memory.  (No
 * counterpart in the reference, whose host closures allocate every buffer
 * with torch on each call.)
 *
 * Some callers of a compiled forward kernel only want its results - an
 * inference server stepping a recurrent layer, a real-time loop, code running
 * under an allocator that forbids cudaMalloc after start-up - yet the kernel
 * also writes training-time scratch (state checkpoints, saved row sums) that
 * such a caller would have to allocate and never read.  This entry point puts
 * those buffers into a static device array owned by the library instead: the
 * caller passes inputs, outputs and the error word as for frnn_launch, and
 * names which kernel parameters are scratch (`scratch_arg[i]`, an index into
 * `args`; what `args` holds at those indices is ignored) and how many bytes
 * each needs (`scratch_bytes[i]`).  Each gets a 256-byte aligned slice.
 *
 * Limits and rules:
 *  - the slices together must fit frnn_static_scratch_capacity() bytes
 *    (32 MiB); a larger request fails with FRNN_E_ARG and launches nothing;
 *  - at most 64 kernel parameters; `nscratch` may not exceed `nargs` and no
 *    parameter index may be listed twice (FRNN_E_ARG otherwise);
 *  - every GPU on which the library is used keeps the array until the process
 *    exits; all calls on a device share it and it keeps the previous call's
 *    contents, so a kernel must not expect zeros there (the forward kernels
 *    only write their scratch) and two calls whose kernels overlap in time on
 *    one GPU race on it - keep them on one stream or serialise them;
 *  - the first call on each device looks the array's device address up
 *    (cudaGetSymbolAddress); make that first call before any stream capture;
 *  - the call itself performs no cudaMalloc / cudaFree and no host heap
 *    allocation.
 */
int frnn_launch_static_scratch(frnn_module_t m, int kernel, const unsigned grid[3], const unsigned block[3],
                               unsigned smem_bytes, void* stream, void* const* args, int nargs,
                               const int* scratch_arg, const size_t* scratch_bytes, int nscratch);

/* Size in bytes of the static scratch array behind frnn_launch_static_scratch. */
size_t frnn_static_scratch_capacity(void);

/* ---- helpers compiled into the library (used by the benchmark harness) ---- */

/* Overwrite `bytes` bytes at `buf` (device) with a byte pattern; writing a
 * buffer larger than L2 between timed iterations evicts the previous
 * iteration's data. */
int frnn_l2_flush(void* buf, size_t bytes, void* stream);

/* Run an FMA-only register-resident loop on every SM for `iters` iterations and
 * return the floating point operations it performs in *flops (2 per FMA).
 * Timed by the caller with events, it measures the FP32 CUDA-core peak that
 * bounds the recurrent kernels.  `sink` is a device buffer of >= 4 bytes. */
int frnn_fp32_peak_probe(float* sink, int iters, void* stream, double* flops);

/*
 * Register-only probe loops of the kinds of FMA the scan kernels execute, one block of 256 threads per SM, timed
 * by the caller like frnn_fp32_peak_probe; *flops receives the operations performed.  `in` is a device buffer of
 * at least 512 floats (small finite values), `sink` one of >= 4 bytes.
 *   kind 0  scalar FFMA, three distinct register operands per instruction
 *   kind 1  scalar FFMA, one operand kept from the previous instruction
 *   kind 2  packed FFMA2, three distinct register pairs
 *   kind 3  packed FFMA2, one pair kept
 *   kind 4  the Delta Rule backward step's seven FMAs per state element (8x8 register tiles, packed)
 *   kind 5  the Delta Rule forward step's three FMAs per state element (4x32 register tile, scalar)
 * The ratio to the peak probe is the share of the FP32 pipe that arithmetic of that kind can reach on this GPU
 * with this compiler; the benchmark reports it beside the kernels' roofline fraction.
 */
int frnn_fp32_mix_probe(int kind, float* sink, const float* in, int iters, void* stream, double* flops);

#ifdef __cplusplus
}
#endif
#endif /* FRNN_H */
