// Host emulation of the few CUDA facilities the generated recurrent kernels
// use, so that the *same generated source* can be compiled with g++ and run on
// the CPU by the test-suite: one OS thread per CUDA thread, std::barrier for
// __syncthreads / warp sync, an exchange buffer for shuffles, memcpy + a
// counter for the TMA bulk copy and its mbarrier.  Test infrastructure only:
// nothing in the library imports or runs this.
#pragma once
#define FRNN_EMU 1
// one OS thread per CUDA thread on a few cores is slow: a bounded device wait must not expire just for that
#define FRNN_WAIT_LIMIT_NS 240000000000ull
#include <atomic>
#include <barrier>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <mutex>
#include <thread>
#include <vector>

typedef unsigned short u16;
typedef unsigned int u32;
typedef unsigned long long u64;
using std::min;
using std::max;

#define FRNN_DEV inline
#define __global__
#define __restrict__
#define __launch_bounds__(...)
#define __align__(n) alignas(n)
// a vector access that is not aligned to its own size faults on the GPU ("misaligned address"); abort here instead
#define FRNN_ASSERT_ALIGNED(p, n) do { if (((uintptr_t)(p)) % (n)) { fprintf(stderr, "emu: misaligned %d-byte access at %p\n", (int)(n), (const void*)(p)); abort(); } } while (0)

struct emu_dim3 { unsigned x = 0, y = 0, z = 0; };
struct emu_cta {
    int nthreads;
    std::barrier<>* block_bar;
    std::vector<std::barrier<>*> warp_bar;
    std::barrier<>* group_bar[16] = {nullptr};   // named barriers, created on first use with that use's thread count
    std::vector<float> xchg;          // [nthreads]
    std::vector<float> tmem;          // Tensor Memory: 128 lanes x 512 columns (allocated on first use)
    int tmem_cols = 0;                // columns the CTA has allocated (0: none)
    unsigned char* smem;
    std::mutex mtx;
};
static thread_local emu_dim3 threadIdx, blockIdx;
static thread_local emu_cta* emu_ctx = nullptr;
static std::mutex emu_atomic_mtx;

#define FRNN_DYN_SMEM(name) unsigned char* name = emu_ctx->smem

FRNN_DEV float emu_u2f(u32 v) { float f; memcpy(&f, &v, 4); return f; }
FRNN_DEV u32 emu_f2u(float f) { u32 v; memcpy(&v, &f, 4); return v; }
FRNN_DEV float frnn_bf16_to_f32(u16 v) { return emu_u2f(((u32)v) << 16); }
FRNN_DEV u16 frnn_f32_to_bf16(float f) {
    u32 x = emu_f2u(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (u16)((x >> 16) | 0x40);  // NaN
    u32 lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (u16)(x >> 16);
}
FRNN_DEV float frnn_f16_to_f32(u16 v) { _Float16 h; memcpy(&h, &v, 2); return (float)h; }
FRNN_DEV u16 frnn_f32_to_f16(float f) { _Float16 h = (_Float16)f; u16 v; memcpy(&v, &h, 2); return v; }

FRNN_DEV u64 frnn_now_ns() {
    return (u64)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// mbarrier emulation inside the 8 bytes: pending transaction bytes (signed), arrivals still expected in this phase,
// the arrival count the barrier was initialised with (15 bits) and the phase parity (1 bit)
struct emu_mbar { int pending; unsigned short remaining; unsigned short count_phase; };
static_assert(sizeof(emu_mbar) == 8, "mbarrier emulation must fit the 64-bit word");
FRNN_DEV void emu_mbar_settle(emu_mbar* b) {
    if (b->remaining == 0 && b->pending == 0) { b->count_phase ^= 1u; b->remaining = (unsigned short)(b->count_phase >> 1); }
}
FRNN_DEV void frnn_mbar_init(u64* bar, u32 count) {
    emu_mbar* b = (emu_mbar*)bar; b->pending = 0; b->remaining = (unsigned short)count; b->count_phase = (unsigned short)(count << 1);
}
FRNN_DEV void frnn_mbar_init_fence() {}
FRNN_DEV void frnn_async_proxy_fence() {}
FRNN_DEV void frnn_mbar_expect_tx(u64* bar, u32 bytes) {
    std::lock_guard<std::mutex> g(emu_ctx->mtx);
    emu_mbar* b = (emu_mbar*)bar;
    if (b->remaining == 0) { fprintf(stderr, "emu: more arrivals on an mbarrier than it was initialised for\n"); abort(); }
    b->pending += (int)bytes; b->remaining--; emu_mbar_settle(b);
}
FRNN_DEV void frnn_mbar_arrive(u64* bar) {
    std::lock_guard<std::mutex> g(emu_ctx->mtx);
    emu_mbar* b = (emu_mbar*)bar;
    if (b->remaining == 0) { fprintf(stderr, "emu: more arrivals on an mbarrier than it was initialised for\n"); abort(); }
    b->remaining--; emu_mbar_settle(b);
}
FRNN_DEV void frnn_bulk_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
    if (((uintptr_t)dst & 15) || ((uintptr_t)src & 15) || (bytes & 15)) {
        fprintf(stderr, "emu: misaligned bulk copy dst=%p src=%p bytes=%u\n", dst, src, bytes); abort();
    }
    memcpy(dst, src, bytes);
    std::lock_guard<std::mutex> g(emu_ctx->mtx);
    emu_mbar* b = (emu_mbar*)bar;
    b->pending -= (int)bytes; emu_mbar_settle(b);
}
// tensor map emulation: the test launcher fills this layout (128 bytes like the real descriptor)
struct alignas(64) frnn_tmap {
    unsigned char* base; u64 dims[4]; u64 strides[3]; u32 box[4]; u32 elt; u32 pad[9];
};
static_assert(sizeof(frnn_tmap) == 128, "tensor map emulation must be 128 bytes");
#define FRNN_TMAP_PARAM const frnn_tmap
FRNN_DEV void frnn_tma_load_4d(void* dst, const frnn_tmap* m, int c0, int c1, int c2, int c3, u64* bar) {
    // a tiled tensor copy wants its shared-memory destination on a 128-byte boundary and the innermost coordinate on 16 bytes
    if (((uintptr_t)dst & 127) || ((long)c0 * m->elt) % 16) { fprintf(stderr, "emu: misaligned tensor load\n"); abort(); }
    unsigned char* d = (unsigned char*)dst;
    size_t total = 0;
    for (u32 w3 = 0; w3 < m->box[3]; w3++)
        for (u32 w2 = 0; w2 < m->box[2]; w2++)
            for (u32 w1 = 0; w1 < m->box[1]; w1++)
                for (u32 w0 = 0; w0 < m->box[0]; w0++) {
                    long i0 = c0 + w0, i1 = c1 + w1, i2 = c2 + w2, i3 = c3 + w3;
                    bool in = i0 >= 0 && i1 >= 0 && i2 >= 0 && i3 >= 0 && (u64)i0 < m->dims[0] && (u64)i1 < m->dims[1] &&
                              (u64)i2 < m->dims[2] && (u64)i3 < m->dims[3];
                    if (in) memcpy(d, m->base + i0 * m->elt + i1 * m->strides[0] + i2 * m->strides[1] + i3 * m->strides[2], m->elt);
                    else memset(d, 0, m->elt);
                    d += m->elt; total += m->elt;
                }
    std::lock_guard<std::mutex> g(emu_ctx->mtx);
    emu_mbar* b = (emu_mbar*)bar;
    b->pending -= (int)total; emu_mbar_settle(b);
}
FRNN_DEV bool frnn_mbar_try(u64* bar, u32 parity) {
    std::lock_guard<std::mutex> g(emu_ctx->mtx);
    emu_mbar* b = (emu_mbar*)bar;
    bool ok = ((b->count_phase & 1u) != parity);
    if (!ok) std::this_thread::yield();
    return ok;
}
FRNN_DEV float frnn_shfl_xor(float v, int off) {
    emu_cta* c = emu_ctx;
    int tid = threadIdx.x, w = tid >> 5;
    c->xchg[tid] = v;
    c->warp_bar[w]->arrive_and_wait();
    float r = c->xchg[tid ^ off];
    c->warp_bar[w]->arrive_and_wait();
    return r;
}
// Tensor Memory emulation: one allocation per CTA starting at column 0; aborts on what the hardware forbids
FRNN_DEV void frnn_tmem_alloc(u32* base_out, u32 ncols) {
    if ((threadIdx.x & 31) != 0) { emu_ctx->warp_bar[threadIdx.x >> 5]->arrive_and_wait(); return; }
    {
        std::lock_guard<std::mutex> g(emu_ctx->mtx);
        if (ncols < 32 || ncols > 512 || (ncols & (ncols - 1)) || emu_ctx->tmem_cols) { fprintf(stderr, "emu: bad Tensor Memory allocation of %u columns\n", ncols); abort(); }
        emu_ctx->tmem.assign(128 * 512, -12345.0f);
        emu_ctx->tmem_cols = (int)ncols;
        *base_out = 0;
    }
    emu_ctx->warp_bar[threadIdx.x >> 5]->arrive_and_wait();
}
FRNN_DEV void frnn_tmem_dealloc(u32 taddr, u32 ncols) {
    if ((threadIdx.x & 31) != 0) return;
    std::lock_guard<std::mutex> g(emu_ctx->mtx);
    if (taddr != 0 || (int)ncols != emu_ctx->tmem_cols) { fprintf(stderr, "emu: Tensor Memory freed with the wrong address or size\n"); abort(); }
    emu_ctx->tmem_cols = 0;
}
FRNN_DEV void frnn_tmem_fence_before_sync() {}
FRNN_DEV void frnn_tmem_fence_after_sync() {}
FRNN_DEV void frnn_tmem_wait_st() {}
FRNN_DEV void frnn_tmem_wait_ld() {}
FRNN_DEV u32 frnn_tmem_lane_base(int warp) { return ((u32)(warp & 3) * 32u) << 16; }
FRNN_DEV float* emu_tmem_at(u32 taddr, int n) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const u32 lane0 = taddr >> 16, col = taddr & 0xffffu;
    if (lane0 != (u32)(warp & 3) * 32u || (int)col + n > emu_ctx->tmem_cols) {
        fprintf(stderr, "emu: Tensor Memory access outside the warp's lanes or the allocation (lane %u col %u n %d)\n", lane0, col, n); abort();
    }
    return &emu_ctx->tmem[(size_t)(lane0 + lane) * 512 + col];
}
#define EMU_TMEM_FN(N) \
    FRNN_DEV void frnn_tmem_st##N(u32 taddr, const float* v) { memcpy(emu_tmem_at(taddr, N), v, 4 * N); } \
    FRNN_DEV void frnn_tmem_ld##N(u32 taddr, float* v) { memcpy(v, emu_tmem_at(taddr, N), 4 * N); }
EMU_TMEM_FN(1) EMU_TMEM_FN(2) EMU_TMEM_FN(4) EMU_TMEM_FN(8) EMU_TMEM_FN(16)
FRNN_DEV int frnn_smem_add(int* p, int v) { std::lock_guard<std::mutex> g(emu_atomic_mtx); int o = *p; *p = o + v; return o; }
template <int N> FRNN_DEV void frnn_regs_release() {}
template <int N> FRNN_DEV void frnn_regs_acquire() {}
FRNN_DEV void frnn_block_sync() { emu_ctx->block_bar->arrive_and_wait(); }
FRNN_DEV void frnn_group_sync(int id, int nthreads) {
    emu_cta* c = emu_ctx;
    {
        std::lock_guard<std::mutex> g(c->mtx);
        if (id < 1 || id > 15 || nthreads % 32) { fprintf(stderr, "emu: bad named barrier %d/%d\n", id, nthreads); abort(); }
        if (!c->group_bar[id]) c->group_bar[id] = new std::barrier<>((std::ptrdiff_t)nthreads);
    }
    c->group_bar[id]->arrive_and_wait();
}
FRNN_DEV void frnn_warp_sync() { emu_ctx->warp_bar[threadIdx.x >> 5]->arrive_and_wait(); }
FRNN_DEV void frnn_atomic_add(float* p, float v) { std::lock_guard<std::mutex> g(emu_atomic_mtx); *p += v; }
FRNN_DEV void frnn_report(int* err, int code) { std::lock_guard<std::mutex> g(emu_atomic_mtx); if (*err == 0) *err = code; }
FRNN_DEV float frnn_expf(float x) { return std::exp(x); }
FRNN_DEV float frnn_logf(float x) { return std::log(x); }
FRNN_DEV float frnn_sqrtf(float x) { return std::sqrt(x); }
struct frnn_pk { float x, y; };
FRNN_DEV frnn_pk frnn_pk_make(float a, float b) { return frnn_pk{a, b}; }
FRNN_DEV frnn_pk frnn_fma2(frnn_pk a, frnn_pk b, frnn_pk c) { return frnn_pk{fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)}; }
FRNN_DEV frnn_pk frnn_mul2(frnn_pk a, frnn_pk b) { return frnn_pk{a.x * b.x, a.y * b.y}; }
FRNN_DEV frnn_pk frnn_add2(frnn_pk a, frnn_pk b) { return frnn_pk{a.x + b.x, a.y + b.y}; }
FRNN_DEV float frnn_rcpf(float x) { return 1.0f / x; }
FRNN_DEV float frnn_divf(float a, float b) { return a / b; }

// ---- launcher -------------------------------------------------------------------
typedef void (*emu_entry_t)(void** args);
static void emu_launch(emu_entry_t fn, const unsigned grid[3], unsigned nthreads, unsigned smem_bytes, void** args) {
    for (unsigned bz = 0; bz < grid[2]; bz++)
        for (unsigned by = 0; by < grid[1]; by++)
            for (unsigned bx = 0; bx < grid[0]; bx++) {
                emu_cta cta;
                cta.nthreads = (int)nthreads;
                std::barrier<> bb((std::ptrdiff_t)nthreads);
                cta.block_bar = &bb;
                std::vector<std::barrier<>*> wb;
                for (unsigned w = 0; w < (nthreads + 31) / 32; w++)
                    wb.push_back(new std::barrier<>((std::ptrdiff_t)std::min(32u, nthreads - w * 32)));
                cta.warp_bar = wb;
                cta.xchg.assign(nthreads, 0.f);
                unsigned char* raw = (unsigned char*)aligned_alloc(128, ((size_t)smem_bytes + 255) / 128 * 128);
                memset(raw, 0xCD, smem_bytes);
                cta.smem = raw;
                std::vector<std::thread> th;
                for (unsigned t = 0; t < nthreads; t++)
                    th.emplace_back([&, t] {
                        threadIdx.x = t; threadIdx.y = threadIdx.z = 0;
                        blockIdx.x = bx; blockIdx.y = by; blockIdx.z = bz;
                        emu_ctx = &cta;
                        fn(args);
                    });
                for (auto& t : th) t.join();
                for (auto* b : wb) delete b;
                for (auto*& gb : cta.group_bar) { delete gb; gb = nullptr; }
                free(raw);
            }
}
