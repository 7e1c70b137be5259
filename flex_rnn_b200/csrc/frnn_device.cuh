// Device-side prelude prepended to every generated recurrent kernel.
//
// The generated kernels are compiled at run time (NVRTC, sm_100a) without any
// include path, so everything they need is defined here: 16-bit float
// conversions, the 1-D TMA bulk copy (cp.async.bulk) with its mbarrier, a
// time-bounded mbarrier wait that reports through an error word instead of
// spinning for ever, and the warp-shuffle row reduction.
//
// When FRNN_EMU is defined the same source is compiled by a host C++ compiler
// against a thread-per-CUDA-thread emulation (tests only); the PTX bodies are
// then replaced by the emulation's definitions of the same functions.
#pragma once

#ifndef FRNN_EMU
typedef unsigned short u16;
typedef unsigned int u32;
typedef unsigned long long u64;
#define FRNN_DEV __device__ __forceinline__
#define FRNN_DYN_SMEM(name) extern __shared__ __align__(128) unsigned char name[]

FRNN_DEV float frnn_bf16_to_f32(u16 v) { return __uint_as_float(((u32)v) << 16); }
FRNN_DEV u16 frnn_f32_to_bf16(float f) {
    u16 r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}
FRNN_DEV float frnn_f16_to_f32(u16 v) {
    float r;
    asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"(v));
    return r;
}
FRNN_DEV u16 frnn_f32_to_f16(float f) {
    u16 r;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}

FRNN_DEV u32 frnn_smem_addr(const void* p) { return (u32)__cvta_generic_to_shared(p); }

FRNN_DEV u64 frnn_now_ns() {
    u64 t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier + TMA bulk copy (global -> shared, no multicast) ------------
FRNN_DEV void frnn_mbar_init(u64* bar, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(frnn_smem_addr(bar)), "r"(count) : "memory");
}
FRNN_DEV void frnn_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
FRNN_DEV void frnn_async_proxy_fence() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
FRNN_DEV void frnn_mbar_expect_tx(u64* bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(frnn_smem_addr(bar)), "r"(bytes) : "memory");
}
// one 1-D bulk copy; dst, src 16-byte aligned, bytes a multiple of 16
FRNN_DEV void frnn_bulk_g2s(void* dst_smem, const void* src_gmem, u32 bytes, u64* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            frnn_smem_addr(dst_smem)),
        "l"(__cvta_generic_to_global(src_gmem)), "r"(bytes), "r"(frnn_smem_addr(bar))
        : "memory");
}
// Tiled TMA load of a 4-D box through a tensor map (cp.async.bulk.tensor, no
// multicast).  The map is encoded on the host (frnn_tensor_map_encode) and
// passed as a __grid_constant__ kernel parameter.  c0 (innermost coordinate)
// times the element size must be a multiple of 16 bytes.
struct __align__(64) frnn_tmap { unsigned long long opaque[16]; };
#define FRNN_TMAP_PARAM const __grid_constant__ frnn_tmap
FRNN_DEV void frnn_tma_load_4d(void* dst_smem, const frnn_tmap* map, int c0, int c1, int c2, int c3, u64* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
            frnn_smem_addr(dst_smem)),
        "l"((u64)map), "r"(frnn_smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
FRNN_DEV bool frnn_mbar_try(u64* bar, u32 parity) {
    u32 ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(frnn_smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// one arrival on an mbarrier that was initialised with a thread count (release semantics at CTA scope:
// the arriving thread's earlier shared-memory writes are visible to whoever sees the phase complete)
FRNN_DEV void frnn_mbar_arrive(u64* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(frnn_smem_addr(bar)) : "memory");
}
// Register reallocation between the warpgroups (4 warps) of a CTA: a warpgroup that needs few registers gives
// some back to the SM's pool, one that needs many takes them.  Executed by all warps of a warpgroup.
template <int N> FRNN_DEV void frnn_regs_release() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> FRNN_DEV void frnn_regs_acquire() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
// barrier over a subset of the CTA's warps (named barrier `id` in 1..15, `nthreads` a multiple of 32)
FRNN_DEV void frnn_group_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
FRNN_DEV float frnn_shfl_xor(float v, int off) { return __shfl_xor_sync(0xffffffffu, v, off); }
FRNN_DEV void frnn_block_sync() { __syncthreads(); }
FRNN_DEV void frnn_warp_sync() { __syncwarp(); }
FRNN_DEV void frnn_atomic_add(float* p, float v) { atomicAdd(p, v); }
// the error word may live in pinned host memory: a plain store reaches it (the first report is kept when it can be)
FRNN_DEV void frnn_report(int* err, int code) {
    if (*(volatile int*)err == 0) *(volatile int*)err = code;
    __threadfence_system();
}
FRNN_DEV float frnn_expf(float x) { return __expf(x); }
FRNN_DEV float frnn_logf(float x) { return __logf(x); }
FRNN_DEV float frnn_sqrtf(float x) { return __fsqrt_rn(x); }
// packed fp32x2 arithmetic (sm_100: one instruction, two lanes)
typedef float2 frnn_pk;
FRNN_DEV frnn_pk frnn_pk_make(float a, float b) { return make_float2(a, b); }
FRNN_DEV frnn_pk frnn_fma2(frnn_pk a, frnn_pk b, frnn_pk c) { return __ffma2_rn(a, b, c); }
FRNN_DEV frnn_pk frnn_mul2(frnn_pk a, frnn_pk b) { return __fmul2_rn(a, b); }
FRNN_DEV frnn_pk frnn_add2(frnn_pk a, frnn_pk b) { return __fadd2_rn(a, b); }
FRNN_DEV float frnn_rcpf(float x) { return __frcp_rn(x); }
FRNN_DEV float frnn_divf(float a, float b) { return __fdividef(a, b); }
// ---- Tensor Memory as on-chip scratch ----------------------------------------------------------
// sm_100 has 256 KB of Tensor Memory per SM (128 lanes x 512 columns of 32 bits) beside the register file and
// shared memory.  It is meant for tensor-core accumulators, but tcgen05.st / tcgen05.ld move plain 32-bit
// registers in and out, so a kernel that never touches the tensor cores can park register tiles there.  Warp w
// of a CTA reaches lanes 32*(w%4) .. 32*(w%4)+31; thread i of the warp owns lane 32*(w%4)+i, and each access
// moves N consecutive columns of that lane.  An address is (lane << 16) | column.
// Allocation (whole CTA, by one warp, a power of two >= 32 columns) blocks while the SM has no room, so a kernel
// must free what it holds on every path out.
FRNN_DEV void frnn_tmem_alloc(u32* base_out_smem, u32 ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(frnn_smem_addr(base_out_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
FRNN_DEV void frnn_tmem_dealloc(u32 taddr, u32 ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
FRNN_DEV void frnn_tmem_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
FRNN_DEV void frnn_tmem_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
FRNN_DEV void frnn_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
FRNN_DEV void frnn_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
FRNN_DEV u32 frnn_tmem_lane_base(int warp) { return ((u32)(warp & 3) * 32u) << 16; }
FRNN_DEV int frnn_smem_add(int* p, int v) { return atomicAdd(p, v); }
FRNN_DEV void frnn_tmem_st1(u32 taddr, const float* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "f"(v[0]) : "memory");
}
FRNN_DEV void frnn_tmem_ld1(u32 taddr, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=f"(v[0]) : "r"(taddr) : "memory");
}
FRNN_DEV void frnn_tmem_st2(u32 taddr, const float* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "f"(v[0]), "f"(v[1]) : "memory");
}
FRNN_DEV void frnn_tmem_ld2(u32 taddr, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "r"(taddr) : "memory");
}
FRNN_DEV void frnn_tmem_st4(u32 taddr, const float* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
}
FRNN_DEV void frnn_tmem_ld4(u32 taddr, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(taddr) : "memory");
}
FRNN_DEV void frnn_tmem_st8(u32 taddr, const float* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}
FRNN_DEV void frnn_tmem_ld8(u32 taddr, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "r"(taddr) : "memory");
}
FRNN_DEV void frnn_tmem_st16(u32 taddr, const float* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(v[8]), "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]) : "memory");
}
FRNN_DEV void frnn_tmem_ld16(u32 taddr, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]) : "r"(taddr) : "memory");
}
#endif  // !FRNN_EMU

// N registers of one thread to / from N consecutive Tensor Memory columns of its lane, in power-of-two pieces
template <int N> FRNN_DEV void frnn_tmem_st(u32 taddr, const float* v) {
    if constexpr (N >= 16) { frnn_tmem_st16(taddr, v); frnn_tmem_st<N - 16>(taddr + 16, v + 16); }
    else if constexpr (N >= 8) { frnn_tmem_st8(taddr, v); frnn_tmem_st<N - 8>(taddr + 8, v + 8); }
    else if constexpr (N >= 4) { frnn_tmem_st4(taddr, v); frnn_tmem_st<N - 4>(taddr + 4, v + 4); }
    else if constexpr (N >= 2) { frnn_tmem_st2(taddr, v); frnn_tmem_st<N - 2>(taddr + 2, v + 2); }
    else if constexpr (N == 1) { frnn_tmem_st1(taddr, v); }
}
template <int N> FRNN_DEV void frnn_tmem_ld(u32 taddr, float* v) {
    if constexpr (N >= 16) { frnn_tmem_ld16(taddr, v); frnn_tmem_ld<N - 16>(taddr + 16, v + 16); }
    else if constexpr (N >= 8) { frnn_tmem_ld8(taddr, v); frnn_tmem_ld<N - 8>(taddr + 8, v + 8); }
    else if constexpr (N >= 4) { frnn_tmem_ld4(taddr, v); frnn_tmem_ld<N - 4>(taddr + 4, v + 4); }
    else if constexpr (N >= 2) { frnn_tmem_ld2(taddr, v); frnn_tmem_ld<N - 2>(taddr + 2, v + 2); }
    else if constexpr (N == 1) { frnn_tmem_ld1(taddr, v); }
}

#ifndef FRNN_WAIT_LIMIT_NS
#define FRNN_WAIT_LIMIT_NS 2000000000ull
#endif

// Bounded wait for a TMA stage.  Returns false (after recording `code` in the
// error word) when the barrier has not completed within the time limit; the
// caller then leaves the kernel, so a lost copy never becomes a hung GPU.
FRNN_DEV bool frnn_mbar_wait(u64* bar, u32 parity, int* err, int code) {
    if (frnn_mbar_try(bar, parity)) return true;
    u64 t0 = frnn_now_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (frnn_mbar_try(bar, parity)) return true;
        if (frnn_now_ns() - t0 > FRNN_WAIT_LIMIT_NS) {
            frnn_report(err, code);
            return false;
        }
    }
}

// ---- checked build (-DFRNN_BOUNDS) ------------------------------------------
// A debugging build of a generated kernel in which every load, store, atomic add
// and 1-D bulk copy first checks that its whole byte range lies inside one of the
// kernel's buffers (the generator registers each pointer parameter with the byte
// extent it derived from the tensor's shape and strides) or inside the CTA's
// dynamic shared memory.  An access outside is not performed: a load yields
// zeros, a store is dropped, and FRNN_ERR_BOUNDS goes to the error word, so that
// an indexing mistake shows up as an error code instead of a memory fault.
// Tiled tensor-map loads need no check (the hardware zero-fills outside the map).
#define FRNN_ERR_BOUNDS 64
#ifdef FRNN_BOUNDS
#define FRNN_BOUNDS_MAX 48
struct frnn_bounds_t {
    const char* lo[FRNN_BOUNDS_MAX];
    const char* hi[FRNN_BOUNDS_MAX];
    const char* smem_lo;
    const char* smem_hi;
    int* err;
    int n;
};
#ifdef FRNN_EMU
static frnn_bounds_t frnn_bounds_state;      // the emulation runs one CTA at a time
#else
__shared__ frnn_bounds_t frnn_bounds_state;  // one table per CTA
#endif
// thread 0 of the CTA, before the first access; the caller synchronises the CTA afterwards
FRNN_DEV void frnn_bounds_begin(int* err, const void* smem, long smem_bytes) {
    frnn_bounds_state.n = 0;
    frnn_bounds_state.err = err;
    frnn_bounds_state.smem_lo = (const char*)smem;
    frnn_bounds_state.smem_hi = (const char*)smem + smem_bytes;
}
FRNN_DEV void frnn_bounds_add(const void* base, long bytes) {
    const int i = frnn_bounds_state.n;
    if (i < FRNN_BOUNDS_MAX && bytes > 0) {
        frnn_bounds_state.lo[i] = (const char*)base;
        frnn_bounds_state.hi[i] = (const char*)base + bytes;
        frnn_bounds_state.n = i + 1;
    }
}
FRNN_DEV bool frnn_access_ok(const void* p, long bytes) {
    const char* a = (const char*)p;
    if (a >= frnn_bounds_state.smem_lo && a + bytes <= frnn_bounds_state.smem_hi) return true;
    for (int i = 0; i < frnn_bounds_state.n; i++)
        if (a >= frnn_bounds_state.lo[i] && a + bytes <= frnn_bounds_state.hi[i]) return true;
    frnn_report(frnn_bounds_state.err, FRNN_ERR_BOUNDS);
    return false;
}
#define FRNN_ACCESS_OK(p, bytes) frnn_access_ok((const void*)(p), (long)(bytes))
#else
#define FRNN_ACCESS_OK(p, bytes) true
#endif
FRNN_DEV void frnn_atomic_add_c(float* p, float v) {
    if (FRNN_ACCESS_OK(p, 4)) frnn_atomic_add(p, v);
}
FRNN_DEV void frnn_bulk_g2s_c(void* dst_smem, const void* src_gmem, u32 bytes, u64* bar) {
    // a refused copy never completes its mbarrier: the waiting side runs into its time limit and leaves
    if (FRNN_ACCESS_OK(src_gmem, bytes) && FRNN_ACCESS_OK(dst_smem, bytes)) frnn_bulk_g2s(dst_smem, src_gmem, bytes, bar);
}
// element i of an array of T, untranslated (the register-prefetched inputs)
template <class T> FRNN_DEV T frnn_ld_raw(const void* p, long i) {
    if (!FRNN_ACCESS_OK((const T*)p + i, sizeof(T))) return T(0);
    return ((const T*)p)[i];
}
template <class T> FRNN_DEV void frnn_st_raw(void* p, long i, T v) {
    if (FRNN_ACCESS_OK((T*)p + i, sizeof(T))) ((T*)p)[i] = v;
}

template <int DT> struct frnn_io;  // 0 = fp32, 1 = bf16, 2 = fp16, 3 = fp64
template <> struct frnn_io<0> {
    typedef float T;
    static FRNN_DEV float ld(const void* p, long i) { return frnn_ld_raw<float>(p, i); }
    static FRNN_DEV void st(void* p, long i, float v) { frnn_st_raw<float>(p, i, v); }
};
template <> struct frnn_io<1> {
    typedef u16 T;
    static FRNN_DEV float ld(const void* p, long i) { return frnn_bf16_to_f32(frnn_ld_raw<u16>(p, i)); }
    static FRNN_DEV void st(void* p, long i, float v) { frnn_st_raw<u16>(p, i, frnn_f32_to_bf16(v)); }
};
template <> struct frnn_io<2> {
    typedef u16 T;
    static FRNN_DEV float ld(const void* p, long i) { return frnn_f16_to_f32(frnn_ld_raw<u16>(p, i)); }
    static FRNN_DEV void st(void* p, long i, float v) { frnn_st_raw<u16>(p, i, frnn_f32_to_f16(v)); }
};
template <> struct frnn_io<3> {
    typedef double T;
    static FRNN_DEV float ld(const void* p, long i) { return (float)frnn_ld_raw<double>(p, i); }
    static FRNN_DEV void st(void* p, long i, float v) { frnn_st_raw<double>(p, i, (double)v); }
};

// sum over the L lanes (L a power of two <= 32) that share one state row
template <int L> FRNN_DEV float frnn_row_sum(float v) {
#pragma unroll
    for (int off = L / 2; off > 0; off >>= 1) v += frnn_shfl_xor(v, off);
    return v;
}

// ---- vector loads / stores with dtype conversion ---------------------------
// frnn_ldv<DT,CNT>(base, i, out): out[0..CNT) = float(base[i .. i+CNT)), where
// the CNT elements are fetched with the widest access their size allows.  The
// caller guarantees that element i sits on a CNT-element boundary of a
// 16-byte aligned base.  Works on shared and global memory alike.
#ifndef FRNN_ASSERT_ALIGNED     // the host emulation defines it to abort on an access the GPU would fault on
#define FRNN_ASSERT_ALIGNED(p, n)
#endif
struct __align__(8) frnn_u2 { u32 x, y; };
struct __align__(16) frnn_u4 { u32 x, y, z, w; };
struct __align__(8) frnn_f2 { float x, y; };
struct __align__(16) frnn_f4 { float x, y, z, w; };

template <int DT> FRNN_DEV float frnn_lo16(u32 w);
template <int DT> FRNN_DEV float frnn_hi16(u32 w);
template <> FRNN_DEV float frnn_lo16<1>(u32 w) { return frnn_bf16_to_f32((u16)(w & 0xffffu)); }
template <> FRNN_DEV float frnn_hi16<1>(u32 w) { return frnn_bf16_to_f32((u16)(w >> 16)); }
template <> FRNN_DEV float frnn_lo16<2>(u32 w) { return frnn_f16_to_f32((u16)(w & 0xffffu)); }
template <> FRNN_DEV float frnn_hi16<2>(u32 w) { return frnn_f16_to_f32((u16)(w >> 16)); }
template <int DT> FRNN_DEV u32 frnn_pack16(float a, float b);
template <> FRNN_DEV u32 frnn_pack16<1>(float a, float b) { return (u32)frnn_f32_to_bf16(a) | ((u32)frnn_f32_to_bf16(b) << 16); }
template <> FRNN_DEV u32 frnn_pack16<2>(float a, float b) { return (u32)frnn_f32_to_f16(a) | ((u32)frnn_f32_to_f16(b) << 16); }

template <int DT> struct frnn_esize { static const int v = DT == 0 ? 4 : (DT == 3 ? 8 : 2); };
template <int DT, int CNT> FRNN_DEV void frnn_ldv(const void* base, long i, float* out) {
#ifdef FRNN_BOUNDS
    if (!FRNN_ACCESS_OK((const char*)base + i * frnn_esize<DT>::v, CNT * frnn_esize<DT>::v)) {
#pragma unroll
        for (int k = 0; k < CNT; k++) out[k] = 0.0f;
        return;
    }
#endif
    if constexpr (DT == 0 && CNT == 4) {
        FRNN_ASSERT_ALIGNED((const float*)base + i, 16);
        frnn_f4 t = *(const frnn_f4*)((const float*)base + i);
        out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
    } else if constexpr (DT == 0 && CNT == 2) {
        FRNN_ASSERT_ALIGNED((const float*)base + i, 8);
        frnn_f2 t = *(const frnn_f2*)((const float*)base + i);
        out[0] = t.x; out[1] = t.y;
    } else if constexpr ((DT == 1 || DT == 2) && CNT == 8) {
        FRNN_ASSERT_ALIGNED((const u16*)base + i, 16);
        frnn_u4 t = *(const frnn_u4*)((const u16*)base + i);
        out[0] = frnn_lo16<DT>(t.x); out[1] = frnn_hi16<DT>(t.x);
        out[2] = frnn_lo16<DT>(t.y); out[3] = frnn_hi16<DT>(t.y);
        out[4] = frnn_lo16<DT>(t.z); out[5] = frnn_hi16<DT>(t.z);
        out[6] = frnn_lo16<DT>(t.w); out[7] = frnn_hi16<DT>(t.w);
    } else if constexpr ((DT == 1 || DT == 2) && CNT == 4) {
        FRNN_ASSERT_ALIGNED((const u16*)base + i, 8);
        frnn_u2 t = *(const frnn_u2*)((const u16*)base + i);
        out[0] = frnn_lo16<DT>(t.x); out[1] = frnn_hi16<DT>(t.x);
        out[2] = frnn_lo16<DT>(t.y); out[3] = frnn_hi16<DT>(t.y);
    } else if constexpr ((DT == 1 || DT == 2) && CNT == 2) {
        FRNN_ASSERT_ALIGNED((const u16*)base + i, 4);
        u32 t = *(const u32*)((const u16*)base + i);
        out[0] = frnn_lo16<DT>(t); out[1] = frnn_hi16<DT>(t);
    } else {
#pragma unroll
        for (int k = 0; k < CNT; k++) out[k] = frnn_io<DT>::ld(base, i + k);
    }
}

template <int DT, int CNT> FRNN_DEV void frnn_stv(void* base, long i, const float* v) {
#ifdef FRNN_BOUNDS
    if (!FRNN_ACCESS_OK((const char*)base + i * frnn_esize<DT>::v, CNT * frnn_esize<DT>::v)) return;
#endif
    if constexpr (DT == 0 && CNT == 4) {
        frnn_f4 t; t.x = v[0]; t.y = v[1]; t.z = v[2]; t.w = v[3];
        FRNN_ASSERT_ALIGNED((float*)base + i, 16);
        *(frnn_f4*)((float*)base + i) = t;
    } else if constexpr (DT == 0 && CNT == 2) {
        frnn_f2 t; t.x = v[0]; t.y = v[1];
        FRNN_ASSERT_ALIGNED((float*)base + i, 8);
        *(frnn_f2*)((float*)base + i) = t;
    } else if constexpr ((DT == 1 || DT == 2) && CNT == 8) {
        frnn_u4 t;
        t.x = frnn_pack16<DT>(v[0], v[1]); t.y = frnn_pack16<DT>(v[2], v[3]);
        t.z = frnn_pack16<DT>(v[4], v[5]); t.w = frnn_pack16<DT>(v[6], v[7]);
        FRNN_ASSERT_ALIGNED((u16*)base + i, 16);
        *(frnn_u4*)((u16*)base + i) = t;
    } else if constexpr ((DT == 1 || DT == 2) && CNT == 4) {
        frnn_u2 t;
        t.x = frnn_pack16<DT>(v[0], v[1]); t.y = frnn_pack16<DT>(v[2], v[3]);
        FRNN_ASSERT_ALIGNED((u16*)base + i, 8);
        *(frnn_u2*)((u16*)base + i) = t;
    } else if constexpr ((DT == 1 || DT == 2) && CNT == 2) {
        FRNN_ASSERT_ALIGNED((u16*)base + i, 4);
        *(u32*)((u16*)base + i) = frnn_pack16<DT>(v[0], v[1]);
    } else {
#pragma unroll
        for (int k = 0; k < CNT; k++) frnn_io<DT>::st(base, i + k, v[k]);
    }
}
