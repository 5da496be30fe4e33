// One-shot all-reduce over peer memory, fused into the epilogue of a row-parallel GEMM.
//
// Replaces "local matmul, then Partial -> all_reduce" of the reference
// (minit/collective/dispatch.py:33-37, minit/collective/tensor.py:72-73, ncclAllReduce at
// minit/nccl/kernel.py:51-53) for outputs of at most 64 rows.
//
// Layout of a rank's symmetric buffer:
//   [0, kArHeaderBytes)   control: word 0 = epoch of the last finished call, word 1 = CTAs done
//   then mailboxes [2 call parities][world senders] of slot_bytes each: 8-byte cells {fp32 partial,
//   epoch} indexed row * N + col, written by the sender with 16-byte stores of two cells.  A cell
//   is valid for a call when its epoch word equals the call's epoch, so data and "ready" travel in
//   one store and the receiver needs no fence and no separate flag.
//
// The thread that holds four finished fp32 partials of a row pushes them into its mailbox in every
// peer's buffer (plain peer stores), then polls -- bounded -- the same cells of the peers'
// mailboxes in its OWN memory and sums over all ranks in rank order: one NVLink crossing per value,
// and every rank adds the same numbers in the same order, so the outputs are bit-identical across
// ranks.  Calls are numbered by a device-side epoch (so a captured graph can be replayed); even and
// odd calls use different mailboxes, and a peer can be at most one call ahead because it needs this
// rank's cells of call e+1 to finish call e+1.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

constexpr int kArMaxWorld = 8;
constexpr size_t kArHeaderBytes = 256;
constexpr size_t kArDataOffset = kArHeaderBytes;

struct ArParams {
    unsigned char* const* peers;   // device array [world]: base of every rank's symmetric buffer (null: no all-reduce)
    unsigned* err;                 // error word: set to 4 when a peer's cells never arrive
    int rank, world;
    size_t slot_bytes;             // bytes of one (parity, sender) mailbox
    int spin_limit;                // polls per peer before the wait gives up (2^22: 0.1 s to a few seconds)
    int two_shot;                  // != 0: a column's partials go to its OWNER rank only, which adds them and sends the sum back
    int cols_per_owner;            // owner of column c = min(c / cols_per_owner, world - 1)
};

__device__ __forceinline__ bool ar_active(const ArParams& a) { return a.world > 1; }

// epoch of the running call: the previous call on this stream has completed, so word 0 is stable
__device__ __forceinline__ unsigned ar_epoch(const ArParams& a) {
    return *reinterpret_cast<volatile unsigned*>(a.peers[a.rank]) + 1u;
}

// Sum v over all ranks.  `cell` = row * N + col of v.x; the four values are adjacent columns.
__device__ __forceinline__ float4 ar_exchange(const ArParams& a, unsigned epoch, size_t cell, float4 v) {
    const int slot = int(epoch & 1u);
    const size_t off = cell * 8;
    const unsigned u0 = __float_as_uint(v.x), u1 = __float_as_uint(v.y), u2 = __float_as_uint(v.z), u3 = __float_as_uint(v.w);
    for (int r = 0; r < a.world; ++r) {
        if (r == a.rank) continue;
        unsigned char* dst = a.peers[r] + kArDataOffset + ((size_t)slot * a.world + a.rank) * a.slot_bytes + off;
        asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(u0), "r"(epoch), "r"(u1), "r"(epoch) : "memory");
        asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 16), "r"(u2), "r"(epoch), "r"(u3), "r"(epoch) : "memory");
    }
    const unsigned char* mine = a.peers[a.rank];
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.world; ++r) {
        if (r == a.rank) { sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w; continue; }
        const unsigned char* src = mine + kArDataOffset + ((size_t)slot * a.world + r) * a.slot_bytes + off;
        uint4 c0, c1;
        int spins = 0;
        for (;;) {
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c0.x), "=r"(c0.y), "=r"(c0.z), "=r"(c0.w) : "l"(src) : "memory");
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c1.x), "=r"(c1.y), "=r"(c1.z), "=r"(c1.w) : "l"(src + 16) : "memory");
            if (c0.y == epoch && c0.w == epoch && c1.y == epoch && c1.w == epoch) break;
            if (++spins > a.spin_limit) { if (a.err) atomicExch(a.err, 4u); break; }   // a peer never arrived: give up, flag the error (the host must read it)
            if (spins > 32) __nanosleep(32);
        }
        sum.x += __uint_as_float(c0.x); sum.y += __uint_as_float(c0.z); sum.z += __uint_as_float(c1.x); sum.w += __uint_as_float(c1.z);
    }
    return sum;
}

// The same exchange for ONE value at a time (a thread that owns a column, not four adjacent ones): one 8-byte cell per
// peer.  Split in two so that a thread with several values first pushes them all and then collects them all: the
// NVLink round trip is paid once, not once per value.
__device__ __forceinline__ void ar_push1(const ArParams& a, unsigned epoch, size_t cell, float v) {
    const int slot = int(epoch & 1u);
    const unsigned u = __float_as_uint(v);
    for (int r = 0; r < a.world; ++r) {
        if (r == a.rank) continue;
        unsigned char* dst = a.peers[r] + kArDataOffset + ((size_t)slot * a.world + a.rank) * a.slot_bytes + cell * 8;
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(u), "r"(epoch) : "memory");
    }
}
__device__ __forceinline__ float ar_pull1(const ArParams& a, unsigned epoch, size_t cell, float v) {
    const int slot = int(epoch & 1u);
    const unsigned char* mine = a.peers[a.rank];
    float sum = 0.f;
    for (int r = 0; r < a.world; ++r) {
        if (r == a.rank) { sum += v; continue; }
        const unsigned char* src = mine + kArDataOffset + ((size_t)slot * a.world + r) * a.slot_bytes + cell * 8;
        uint2 c;
        int spins = 0;
        for (;;) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(c.x), "=r"(c.y) : "l"(src) : "memory");
            if (c.y == epoch) break;
            if (++spins > a.spin_limit) { if (a.err) atomicExch(a.err, 4u); break; }   // a peer never arrived: give up, flag the error (the host must read it)
            if (spins > 32) __nanosleep(32);
        }
        sum += __uint_as_float(c.x);
    }
    return sum;
}

// ar_pull1 for NR rows of one column at once (cells cell0, cell0 + stride, ...): the NR cells of a peer are loaded
// together, so a group of rows costs one trip to memory per peer instead of one per value (a thread that collects 32 rows
// from 3 peers one value at a time spends 32 x 3 x ~0.7 us in dependent loads).  v[j] holds this rank's partial on entry
// and the sum over all ranks, added in rank order, on return; rows j >= nrows are left alone.
template <int NR>
__device__ __forceinline__ void ar_pull_rows(const ArParams& a, unsigned epoch, size_t cell0, size_t stride, int nrows, float (&v)[NR]) {
    const int slot = int(epoch & 1u);
    const unsigned char* mine = a.peers[a.rank];
    float sum[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) sum[j] = 0.f;
    for (int r = 0; r < a.world; ++r) {
        if (r == a.rank) {
#pragma unroll
            for (int j = 0; j < NR; ++j) sum[j] += v[j];
            continue;
        }
        const unsigned char* src = mine + kArDataOffset + ((size_t)slot * a.world + r) * a.slot_bytes + cell0 * 8;
        uint2 c[NR];
        int spins = 0;
        for (;;) {
            bool all = true;
#pragma unroll
            for (int j = 0; j < NR; ++j)
                if (j < nrows) asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(c[j].x), "=r"(c[j].y) : "l"(src + (size_t)j * stride * 8) : "memory");
#pragma unroll
            for (int j = 0; j < NR; ++j)
                if (j < nrows) all = all && c[j].y == epoch;
            if (all) break;
            if (++spins > a.spin_limit) { if (a.err) atomicExch(a.err, 4u); break; }   // a peer never arrived: give up, flag the error (the host must read it)
            if (spins > 32) __nanosleep(32);
        }
#pragma unroll
        for (int j = 0; j < NR; ++j)
            if (j < nrows) sum[j] += __uint_as_float(c[j].x);
    }
#pragma unroll
    for (int j = 0; j < NR; ++j)
        if (j < nrows) v[j] = sum[j];
}

// Two-shot form for batches of several rows.  The one-shot exchange above sends every value to every peer: (world - 1) x
// the bytes of the result, 14.7 MB per rank at 32 rows x 8192 columns on 8 ranks.  Here the ranks split the columns: a
// rank sends its partial of a column to the column's owner only; the owner adds all ranks' partials in rank order (its own
// in its place) and sends the sum to everyone, so every rank holds the same bits.  2 x (world - 1) / world of the result's
// bytes per rank and two NVLink crossings per value instead of one.  The cells are the same mailboxes: partials land in
// the OWNER's buffer in the sender's mailbox (where ar_pull1 looks), the sum in every peer's buffer in the owner's
// mailbox; a rank writes only its own mailbox in anybody's buffer, and the columns it owns and the columns it does not
// are different cells, so the two phases never meet.
__device__ __forceinline__ int ar_owner(const ArParams& a, int col) {
    const int o = col / a.cols_per_owner;
    return o < a.world ? o : a.world - 1;
}
__device__ __forceinline__ void ar_push_to(const ArParams& a, unsigned epoch, int dst_rank, size_t cell, float v) {
    const int slot = int(epoch & 1u);
    unsigned char* dst = a.peers[dst_rank] + kArDataOffset + ((size_t)slot * a.world + a.rank) * a.slot_bytes + cell * 8;
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ float ar_read_from(const ArParams& a, unsigned epoch, int src_rank, size_t cell) {
    const int slot = int(epoch & 1u);
    const unsigned char* src = a.peers[a.rank] + kArDataOffset + ((size_t)slot * a.world + src_rank) * a.slot_bytes + cell * 8;
    uint2 c;
    int spins = 0;
    for (;;) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(c.x), "=r"(c.y) : "l"(src) : "memory");
        if (c.y == epoch) break;
        if (++spins > a.spin_limit) { if (a.err) atomicExch(a.err, 4u); break; }   // the owner never answered: give up, flag the error
        if (spins > 32) __nanosleep(32);
    }
    return __uint_as_float(c.x);
}

// Called by ONE thread of every CTA of the grid, after the CTA's last exchange: the last CTA to
// leave publishes the epoch for the next call.
__device__ __forceinline__ void ar_leave(const ArParams& a, unsigned epoch, unsigned total_ctas) {
    unsigned* ctl = reinterpret_cast<unsigned*>(a.peers[a.rank]);
    __threadfence();
    if (atomicAdd(ctl + 1, 1u) == total_ctas - 1) { ctl[1] = 0; __threadfence(); *reinterpret_cast<volatile unsigned*>(ctl) = epoch; }
}

}  // namespace mt
