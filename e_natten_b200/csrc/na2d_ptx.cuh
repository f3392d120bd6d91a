// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, no multicast),
// tcgen05 (TMEM allocation, UMMA issue / commit, TMEM loads) and the descriptor encodings.
//
// Every wait is bounded: when the limit runs out the waiter records a code in the device error
// word, raises the CTA-wide abort flag and carries on, so that a kernel can never spin for ever;
// the host reads the word with na2d_check() or na2d_poll().
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace na2d_ptx {

enum : unsigned int {
    kErrLoadWait = 1u,      // a TMA load barrier did not complete
    kErrMmaWait = 2u,       // an MMA commit barrier did not complete
    kErrOther = 4u,
    kErrSmemBase = 8u       // the dynamic shared memory did not start on a 1024-byte boundary
};

// A waiting thread is suspended by the hardware inside mbarrier.try_wait for up to kWaitHintNs
// (a hint; the hardware may return earlier), so that waiting warps leave the issue slots of their
// SM sub-partition to the warps that work (the MMA-issue warp shares its scheduler with softmax
// warps).
// A wait is bounded by real time (kWaitLimitNs), not by a number of polls alone: under a profiler
// a replay pass that instruments the kernel runs the working warps orders of magnitude slower,
// and a bound counted in plain polling rounds (as it once was) ran out there although nothing
// was stuck.  Once the CTA has aborted, later waits end after their polling stage.
constexpr uint32_t kWaitHintNs = 1000;
constexpr unsigned long long kWaitLimitNs = 4000000000ull;   // 4 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// What a bounded wait needs to report that it gave up, kept in shared memory (one per CTA, set up
// by one thread before the first wait) so that a waiting thread carries a single pointer: the abort
// flag (set by the first waiter that gives up, it shortens every later wait of the CTA), the device
// error word the host reads with na2d_check / na2d_poll, and the time limit of one wait.
struct WaitState {
    uint32_t abort;
    uint32_t limit_us;       // microseconds a wait may last
    unsigned int* err_word;
};
struct WaitCtx {
    WaitState* st;
};
// (accessors in the shared state space: a 32-bit address, no generic pointer kept in registers)
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.volatile.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void wait_state_init(WaitState* st, unsigned int* err_word, unsigned long long limit_ns) {
    st->abort = 0;
    // err_word[1], when set, overrides the limit (microseconds)
    const uint32_t configured = err_word[1];
    st->limit_us = configured != 0u ? configured : static_cast<uint32_t>(limit_ns / 1000ull);
    st->err_word = err_word;
}

// ------------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return done != 0;
}
// Non-blocking test of a phase (for a thread that polls more than one barrier).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait.  Returns false if the wait gave up (after recording `err_code`).
//
// Three stages.  (1) One try_wait, which the hardware may hold for up to kWaitHintNs: most waits
// end here.  (2) A plain polling loop of kPollRounds rounds.  (3) A wait that is still open after
// that (about a millisecond) sleeps a microsecond between its polls and counts them: k rounds
// mean that at least k microseconds of real time have passed, whatever slows the warps down, so
// the count is the clock, and the wait gives up when it reaches the limit (or when the CTA has
// aborted meanwhile).  None of the stages keeps anything alive but a counter: a waiting warp
// usually sits among code with every register in use, and whatever a wait needed beyond that
// (a 64-bit start time, say) would be spilled and reloaded around every wait that lasts - which
// was measured as several per cent of the kernels' time.
constexpr uint32_t kPollRounds = 1024;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& wc, unsigned int err_code) {
    if (mbar_try_wait(bar, parity)) return true;              // common case: already complete
#pragma unroll 1
    for (uint32_t i = 0; i < kPollRounds; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint32_t st = smem_u32(wc.st);                      // {abort, limit_us, err_word}
#pragma unroll 1
    for (uint32_t i = 0; i < ld_shared_u32(st + 4) && ld_shared_u32(st) == 0; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(1000);
    }
    st_shared_u32(st, 1u);
    atomicOr(wc.st->err_word, err_code);
    return false;
}

// Book-keeping of a TMA producer: which load barriers it has armed last, so that a producer that
// stops early (a wait for a free buffer gave up) can wait for the loads it has in flight before
// the CTA exits - a bulk copy must not land in shared memory that no longer belongs to the CTA.
// All of a kernel's barriers sit in one array; a barrier is known here by its index in it, and the
// state is two bit masks (armed, parity of the armed phase), so nothing leaves the registers.
struct LoadTracker {
    uint64_t* base;          // the kernel's barrier array (at most 32 entries)
    uint32_t armed = 0, par = 0;
    bool ok = true;
    __device__ __forceinline__ explicit LoadTracker(uint64_t* bars) : base(bars) {}
    // waits (bounded) until `empty` says the buffer is free; false once any wait has given up
    __device__ __forceinline__ bool acquire(uint64_t* empty, uint32_t parity, const WaitCtx& wc) {
        if (ok) ok = mbar_wait(empty, parity, wc, kErrLoadWait);
        return ok;
    }
    __device__ __forceinline__ void arm(uint64_t* full, uint32_t parity, uint32_t bytes) {
        const uint32_t bit = 1u << static_cast<uint32_t>(full - base);
        armed |= bit;
        par = parity ? (par | bit) : (par & ~bit);
        mbar_expect_tx(full, bytes);
    }
    // only after a give-up: every armed barrier completes when its bytes have landed
    __device__ __forceinline__ void drain(const WaitCtx& wc) {
        if (ok) return;
        for (uint32_t s = 0; s < 32; ++s)
            if ((armed >> s) & 1u) mbar_wait(base + s, (par >> s) & 1u, wc, kErrLoadWait);
    }
};

// Generic-proxy writes to shared memory become visible to the async proxy (TMA, UMMA).
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------------ TMA
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 5-D tiled load global -> shared, completion on an mbarrier of this CTA.  No multicast.
// Coordinates are (channel, column, row, head, batch); the channel coordinate times the element
// size must be a multiple of 16 bytes.  Loads may start outside the tensor (the box is filled
// with zeros there).
__device__ __forceinline__ void tma_load_5d(void* dst, const void* tmap, uint64_t* bar,
                                            int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// The same box brought into L2 only: nothing is written to shared memory and nothing signals
// completion.  A producer issues it for a box it cannot load yet (its shared-memory buffer is
// still being read), so that the load proper finds the data in L2.  Same coordinate rules.
__device__ __forceinline__ void tma_prefetch_5d(const void* tmap, int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.prefetch.tensor.5d.L2.global.tile [%0, {%1, %2, %3, %4, %5}];"
        ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// 5-D tiled store shared -> global (bulk async-group completion).  Pixels of the box that lie
// outside the tensor are not written.  Coordinates must not be negative; c0 as for loads.
__device__ __forceinline__ void tma_store_5d(const void* tmap, uint32_t smem_src, int c0, int c1, int c2, int c3,
                                             int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Waits until at most N of this thread's bulk groups are still incomplete (writes performed).
template <int N>
__device__ __forceinline__ void bulk_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------------------------ tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(slot_in_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (row = lane, two
// 16-bit K elements per 32-bit column).
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One lane of a converged warp, chosen by the hardware.  Issue code guarded by this predicate
// compiles to a much shorter instruction sequence per tcgen05.mma than the same code guarded by
// `lane == 0` (measured on B200: ~35 against ~60 cycles per MMA for the issuing thread, which is
// what bounds MMAs with N < 128): the compiler knows that a single thread runs it.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}
// The same two, predicated inside the instruction stream instead of by a branch around them: the
// whole warp runs the issue loop with warp-uniform control flow and operands, and `issue` (true in
// one lane) decides who executes the instruction.  A `tcgen05.mma` takes its descriptors from
// uniform registers; operands computed under a divergent branch have to be moved there one by
// one, which was measured at ~85 cycles per MMA whatever its shape.
__device__ __forceinline__ void umma_ss_if(uint32_t issue, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}
__device__ __forceinline__ void umma_ts_if(uint32_t issue, uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}
__device__ __forceinline__ void umma_commit_if(uint32_t issue, uint64_t* bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n"
        ::"r"(smem_u32(bar)), "r"(issue) : "memory");
}
// The mbarrier gets one arrival when every UMMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 8 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x4(uint32_t taddr, const uint32_t (&r)[4]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// Register re-balancing between warpgroups (all four warps of an aligned group of four must
// execute it): the data-movement / MMA-issue group gives registers up, the softmax groups take them.
template <int N> __device__ __forceinline__ void reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
// Named barrier among `nthreads` threads (ids 1..15; 0 is __syncthreads).
__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Store counterpart of tmem_ld_32x32.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// ------------------------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor (64 bit) for a swizzled canonical layout.
//   bits  0-13  start address >> 4          bits 16-29  leading byte offset >> 4
//   bits 32-45  stride byte offset >> 4     bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  swizzle: 2 = 128 B, 4 = 64 B
// K-major operand: rows of `row_bytes` (= swizzle span), 8-row groups `sbo` bytes apart.
// MN-major operand: the same storage read transposed; `lbo` = distance between swizzle-span
// wide slabs along MN, `sbo` = distance between 8-row groups along K.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t swizzle_code) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(swizzle_code & 7u) << 61;
    return d;
}

// The same descriptor split into its two 32-bit words: the high word is a constant of the
// operand kind, the low word carries the address, so stepping along K is one 32-bit add
// (2 per 32 bytes) on the low word - cheap enough for the single thread that issues the MMAs.
__device__ __forceinline__ constexpr uint32_t smem_desc_hi(uint32_t sbo_bytes, uint32_t swizzle_code) {
    return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | ((swizzle_code & 7u) << 29);
}
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint64_t desc64(uint32_t hi, uint32_t lo) {
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

// Instruction descriptor for kind::f16 (fp16 / bf16 inputs, fp32 accumulate).
//   bits 4-5 D format (1 = f32); 7-9 A format, 10-12 B format (0 = f16, 1 = bf16);
//   bit 15 A major, bit 16 B major (0 = K-major, 1 = MN-major); 17-22 N >> 3; 24-28 M >> 4.
// A and B carry their own format fields, but they must name the same type: an fp16 A with a
// bf16 B raises an illegal-instruction fault on B200.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool a_bf16, bool b_bf16, bool a_mn_major,
                                                  bool b_mn_major) {
    return (1u << 4) | ((a_bf16 ? 1u : 0u) << 7) | ((b_bf16 ? 1u : 0u) << 10) |
           ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace na2d_ptx
