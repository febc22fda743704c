// Block-sparse matmul on 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory) for fp16 / bf16 / fp32 (as TF32) data and block sizes 64 and 128.
//
// The work list is a step plan (plan_panel.cu): the output blocks of one output row are grouped
// into panels of G (1 or 2) blocks; a step is one inner index t whose A block exists and that
// hits at least one B block of the panel.  Per step one A block and the step's B blocks are
// staged; the B blocks of neighbouring panel columns lie side by side in shared memory, so a run
// of present columns is multiplied by ONE tcgen05.mma of N = run x bs, and the A block is fetched
// once per step instead of once per (A, B) pair.  With G = 1 a step is a single (A, B) pair.
//
// A ring entry is one (step, k-chunk): KE = 64 (16-bit data) or 32 (fp32) of the bs contraction
// indices of the step's blocks, 128 bytes of a K-major row, so that the MMAs of the first chunk can
// start while the next is in flight.  A block read K-major contributes its KE-column piece k
// (bs rows x 128 B); a block read MN-major contributes rows [KE k, KE k + KE) as bs/KE sub-tiles of
// KE rows x 128 B.  The
// transposed products of the backward pass (BSP_OP_NT, BSP_OP_TN) use the same staged data;
// only the major-ness bits of the shared-memory and instruction descriptors change.
//
// Persistent CTAs (1 to 3 per SM) of S + 5 warps, S = ring stages:
//   warps 0..S-1  producers: warp w owns ring stage w; one lane polls that stage's "empty"
//                 barrier and issues the TMA copies of its entries (128-byte swizzle) as soon as
//                 the stage is free, so the copies of different stages issue in parallel
//   warp S        MMA issuer: converged warp, one elected lane issues four tcgen05.mma (K = 16
//                 each) per run and entry, releases the stage with tcgen05.commit, and hands a
//                 finished accumulator group (the G accumulators of a panel, adjacent
//                 tensor-memory columns) to the epilogue
//   warps S+1..S+4 epilogue: tcgen05.ld the fp32 accumulators, hand the accumulator group back as
//                 soon as the last of them is in registers, apply the epilogue variant (plain;
//                 bias row added; or scale + block-local softmax: exp(s - row maximum) and the
//                 (maximum, sum) pair of every row), convert, exchange words between lanes so
//                 that neighbouring lanes hold neighbouring bytes of one output row, and store
//                 whole 128-byte lines; blocks no step touched are written as zeros (the bias
//                 row; ones in softmax mode)
//
// The panels are cut into small units that are handed out in order: a CTA starts with unit
// blockIdx.x and then draws unit numbers from a global counter (or, without one, takes every
// gridDim.x-th unit).  Producer 0 draws two units ahead and publishes the numbers through a
// queue in shared memory, from which all roles of the CTA read the same sequence.
//
// Every mbarrier and queue wait is bounded (about one second): a wait that runs out records
// BSP_ERR_DEVICE_TIMEOUT in the status word, all roles leave their loops, outstanding copies
// and MMAs are drained with bounded waits, tensor memory is freed and the kernel returns.
// (tcgen05.alloc itself blocks while CTAs of an earlier grid on the same SM still hold tensor
// memory, and returns when they exit.)
#include <float.h>

#include <atomic>

#include "common.cuh"
#include "umma_common.cuh"

namespace bsp {

using namespace umma;

namespace {

constexpr uint32_t kCtrlLast = 0x100u;
// Slots of the per-CTA queue of unit numbers (dynamic scheduling).
constexpr int kUnitQueue = 8;

// Per (block size, panel width): ring depth, accumulator groups (of G x bs tensor-memory
// columns each) and resident CTAs per SM.  Shared memory: stages x (1 + G) x bs x 128 bytes.
template <int BS, int G> struct PCfg;
template <> struct PCfg<64, 1> {   // 3 x (4 x 16 KiB), 3 x 128 columns
    static constexpr int kStages = 4, kGroups = 2, kCtasPerSm = 3, kThreads = 32 * (kStages + 5);
};
template <> struct PCfg<64, 2> {   // 2 x (4 x 24 KiB), 2 x 256 columns
    static constexpr int kStages = 4, kGroups = 2, kCtasPerSm = 2, kThreads = 32 * (kStages + 5);
};
template <> struct PCfg<128, 1> {  // 6 x 32 KiB, 4 x 128 columns
    static constexpr int kStages = 6, kGroups = 4, kCtasPerSm = 1, kThreads = 32 * (kStages + 5);
};
template <> struct PCfg<128, 2> {  // 4 x 48 KiB, 2 x 256 columns
    static constexpr int kStages = 4, kGroups = 2, kCtasPerSm = 1, kThreads = 32 * (kStages + 5);
};

constexpr int tmem_cols_pow2(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

template <int BS, int G>
struct PSmem {
    static constexpr int kChunkBytes = BS * 128;           // one block's share of a ring entry: bs x 64 elements
    static constexpr int kStageBytes = (1 + G) * kChunkBytes;
    static constexpr int kDataBytes = PCfg<BS, G>::kStages * kStageBytes;
    static constexpr int kBarBytes = (2 * PCfg<BS, G>::kStages + 2 * PCfg<BS, G>::kGroups + 1) * 8;
    static constexpr int kMiscBytes = (2 * PCfg<BS, G>::kStages + 2 + kUnitQueue + 5) * 4;
    static constexpr int kTotal = kDataBytes + kBarBytes + kMiscBytes + 1024;
};

// Shared-memory matrix descriptors of a ring entry (all 128-byte swizzle, 8-row groups 1024 B
// apart).  K-major: rows are M/N indices, 16 contraction elements = 32 bytes along the row.
// MN-major: rows are contraction indices (16 rows = 2048 B per MMA), the M/N extent is cut
// into 64-wide atoms of 64 rows x 128 B = 8 KiB, `LBO` apart.
// fp32 operands (TF32): an MMA takes 8 contraction elements = again 32 bytes K-major; MN-major it
// takes 8 rows = 1024 B, the atoms are 32 rows x 128 B = 4 KiB with 4-row groups 512 B apart and
// the swizzle works on 32-byte granules (layout type 1).
template <typename T, bool MN_MAJOR>
__device__ __forceinline__ uint64_t chunk_desc(uint32_t base, int kk) {
    if (MN_MAJOR) {
        if (sizeof(T) == 4) return make_smem_desc(base + kk * 1024, 4096, 512, 1);
        return make_smem_desc(base + kk * 2048, 8192, 1024);
    }
    return make_smem_desc(base + kk * 32, 16, 1024);
}

// One MMA of the element type's kind, issued by the elected lane of a converged warp.
template <typename T>
__device__ __forceinline__ void tc_mma_elect(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    if (sizeof(T) == 4) tc_mma_tf32_elect(d_tmem, adesc, bdesc, idesc, accumulate);
    else tc_mma_f16_elect(d_tmem, adesc, bdesc, idesc, accumulate);
}

// Softmax epilogue, block size 128 (lane = accumulator row): the maximum of scale * x over the row's
// 128 columns, read from tensor memory ahead of the pass that exponentiates.
__device__ __forceinline__ float row_max_scaled(uint32_t taddr, float scale) {
    float m = -FLT_MAX;
#pragma unroll
    for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t v[32];
        tc_ld32(taddr + c0, v);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) m = fmaxf(m, __uint_as_float(v[e]) * scale);
    }
    return m;
}

// Exchange inside a quad (lanes 4r .. 4r + 3).  In: thread q holds words w[g], g = 0..7, where word (g, q)
// lies at byte 16 g + 4 q of a 128-byte row.  Out: thread q holds the eight words of bytes
// [32 q, 32 q + 32): the word at byte 32 q + 4 j is in slot {0, 2, 4, 6, 1, 3, 5, 7}[j].  Two butterfly
// stages; a stage pairs lane bit m with slot bit sb: a thread keeps the slots whose bit equals its own
// and trades the others with its partner, the received word taking the vacated slot.
__device__ __forceinline__ void quad_gather8(uint32_t (&w)[8], int lane) {
#pragma unroll
    for (int stage = 0; stage < 2; ++stage) {
        const int m = stage == 0 ? 2 : 1, sb = stage == 0 ? 4 : 2;
        const bool up = (lane & m) != 0;
#pragma unroll
        for (int s0 = 0; s0 < 8; ++s0) {
            if (s0 & sb) continue;
            const int s1 = s0 | sb;
            const uint32_t r = __shfl_xor_sync(0xffffffffu, up ? w[s0] : w[s1], m);
            if (up) w[s0] = r; else w[s1] = r;
        }
    }
}

// Exchange among the 8 lanes of a group (lanes 8 m .. 8 m + 7).  In: lane l holds 8 chunks of 4 words,
// chunk c of its own row at w[4 c ..].  Out: slot i holds chunk (l & 7) of the row of lane (l & ~7) + i.
// Three butterfly stages over lane bits 4, 2, 1 (slot bit = lane bit), as in quad_gather8.
__device__ __forceinline__ void octet_gather_chunks(uint32_t (&w)[32], int lane) {
#pragma unroll
    for (int stage = 0; stage < 3; ++stage) {
        const int m = 4 >> stage;
        const bool up = (lane & m) != 0;
#pragma unroll
        for (int s0 = 0; s0 < 8; ++s0) {
            if (s0 & m) continue;
            const int s1 = s0 | m;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t r = __shfl_xor_sync(0xffffffffu, up ? w[4 * s0 + k] : w[4 * s1 + k], m);
                if (up) w[4 * s0 + k] = r; else w[4 * s1 + k] = r;
            }
        }
    }
}

// What the epilogue does besides converting and storing the accumulators.
constexpr int kEpiPlain = 0;    // nothing
constexpr int kEpiBias = 1;     // adds the bias row of the block's column (the linear helper)
constexpr int kEpiSoftmax = 2;  // scaled scores -> exp(s - row maximum inside the block), plus (maximum, sum) per row

template <typename T, int BS, int OP, int G, int EPI>
__global__ void __launch_bounds__(PCfg<BS, G>::kThreads, PCfg<BS, G>::kCtasPerSm)
matmul_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   int64_t n_a, int64_t n_b, T* __restrict__ out,
                   const T* __restrict__ bias, const int64_t* __restrict__ out_lut,
                   float scale, float2* __restrict__ stats,
                   const int32_t* __restrict__ panel_first, const int32_t* __restrict__ step_off,
                   const int32_t* __restrict__ steps, const int32_t* __restrict__ touched,
                   const int32_t* __restrict__ unit_panel, const int32_t* __restrict__ unit_step,
                   int n_units, uint32_t idesc_no_n, int32_t* __restrict__ sched,
                   int32_t* __restrict__ status_word) {
    using C = PCfg<BS, G>;
    using L = PSmem<BS, G>;
    // A ring entry holds KE contraction indices (128 bytes of a K-major row): 64 for 16-bit data, 32 for
    // fp32; a block read MN-major is staged as BS / KE atoms of KE rows x 128 bytes.
    constexpr int KE = 128 / (int)sizeof(T), ATOM = KE * 128;
    constexpr int S = C::kStages, NG = C::kGroups, H = BS / KE, KC = BS / KE;
    constexpr bool A_MN = (OP == BSP_OP_TN);
    constexpr bool B_MN = (OP != BSP_OP_NT);
    constexpr bool BIAS = EPI == kEpiBias, SOFTMAX = EPI == kEpiSoftmax;
    constexpr int TMEM_COLS = tmem_cols_pow2(NG * G * BS);
    static_assert(S <= 32 && G <= 4 && G * BS <= 256, "panel configuration out of range");

    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t data = (raw + 1023u) & ~1023u;
    unsigned char* data_ptr = smem_raw + (data - raw);
    const uint32_t bars = data + L::kDataBytes;
    const uint32_t full_bar = bars, empty_bar = bars + 8 * S, tfull_bar = bars + 16 * S,
                   tempty_bar = tfull_bar + 8 * NG, drain_bar = tempty_bar + 8 * NG;
    volatile uint32_t* ctrl_slot = reinterpret_cast<volatile uint32_t*>(data_ptr + L::kDataBytes + L::kBarBytes);
    volatile int* armed = reinterpret_cast<volatile int*>(ctrl_slot + S);
    volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(armed + S);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    volatile int* unit_q = abort_flag + 1;          // unit numbers, slot = position in this CTA's sequence % kUnitQueue
    volatile int* q_tail = unit_q + kUnitQueue;     // positions published so far
    volatile int* q_heads = q_tail + 1;             // per epilogue warp: positions retired
    const bool dyn = sched != nullptr;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Programmatic dependent launch: a following launch of this kernel may move its CTAs onto the
    // SMs as ours leave and run its set-up (barriers, tensor-memory allocation) meanwhile; it
    // does not touch global memory before its own griddepcontrol.wait below, which returns when
    // this grid has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
            armed[s] = -1;
        }
        for (int i = 0; i < NG; ++i) {
            mbar_init(tfull_bar + 8 * i, 1);
            mbar_init(tempty_bar + 8 * i, 4);
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        unit_q[0] = (int)blockIdx.x < n_units ? (int)blockIdx.x : -1;
        *q_tail = 1;
        for (int i = 0; i < 4; ++i) q_heads[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    if (warp == S) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr((const void*)tmem_base_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    // everything the previous kernels of the stream wrote is visible after this
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // Work is dealt in units (contiguous panel ranges of about equal cost).  Every CTA starts with
    // unit blockIdx.x.  Static schedule (sched == nullptr): it goes on with blockIdx.x + gridDim.x,
    // ...  Dynamic schedule: the CTA's later units come from a global counter (sched[0]), so a CTA
    // that falls behind (slower path to L2 / HBM, an unlucky run of heavy panels) simply takes fewer
    // of them.  Either way the units are handed out in order, so all CTAs sweep the output together
    // and the operand blocks of one batch stay in L2 while they are in use.
    // The CTA's sequence of units goes through a small queue in shared memory: producer 0 fetches
    // the next number one unit ahead of its own progress and publishes it; every role reads
    // position n of the sequence with unit_at(n).  -1 ends the sequence.
    // The i-th ring entry of the CTA's whole sequence uses stage i % S; a stage's barrier parity is
    // its use count.
    auto unit_at = [&](int n, bool block) -> int {  // -2: not published yet (only if !block)
        if (!dyn) {
            const long long u = (long long)blockIdx.x + (long long)n * gridDim.x;
            return u < n_units ? (int)u : -1;
        }
        if (*q_tail <= n) {
            if (!block) return -2;
            unsigned long long t0 = 0;
            for (uint32_t spins = 1; *q_tail <= n; ++spins) {
                if ((spins & 0x3f) == 0) {
                    if (t0 == 0) t0 = global_timer();
                    if (*abort_flag || global_timer() - t0 > kWaitLimitNs) {
                        *abort_flag = 1;
                        if (status_word) *status_word = BSP_ERR_DEVICE_TIMEOUT;
                        return -1;
                    }
                }
            }
        }
        __threadfence_block();
        return unit_q[n % kUnitQueue];
    };
    if ((int)blockIdx.x < n_units) {
        if (warp < S) {
            // ---------------- producers: warp w owns ring stage w ----------------
            // ring entry = (step, k-chunk); absolute entry index = step * KC + k-chunk.  Producer w
            // fills the entries whose position in the CTA's sequence is w mod S; every producer is a warp of its own (one lane
            // active), so the stages are refilled independently and the copy instructions of
            // different stages issue in parallel.
            if (lane == 0) {
                const int slot = warp;
                const int4* recs = reinterpret_cast<const int4*>(steps);
                auto range_of = [&](int uu, int& b, int& e) {
                    if (uu >= 0) {
                        b = unit_step[uu] * KC;
                        e = unit_step[uu + 1] * KC;
                    } else {
                        b = e = 0;
                    }
                };
                auto load_rec = [&](int e, int4& r0, int4& r1) {
                    const int64_t i = e / KC;
                    r0 = recs[2 * i];
                    r1 = recs[2 * i + 1];
                };
                // Producer 0 of a dynamically scheduled CTA also feeds the unit queue.  It draws a
                // number from the global counter, lets the answer travel while it issues two more
                // copies, then publishes it; it keeps the queue two positions ahead of its own unit.
                const bool scheduler = dyn && slot == 0;
                int m_pub = 1;             // next queue position to publish
                int pend = 0;              // counter value drawn for it
                int pend_age = 0;          // copies issued since the draw
                bool pend_valid = false, closed = false;  // closed: the end marker is published
                bool alive = true;
                auto draw = [&]() {
                    pend = atomicAdd(sched, 1);
                    pend_valid = true;
                    pend_age = 0;
                };
                auto publish = [&]() {
                    // the slot was last used by position m_pub - kUnitQueue: all epilogue warps must be past it
                    unsigned long long t0 = 0;
                    for (uint32_t spins = 1;; ++spins) {
                        const int head = min(min(q_heads[0], q_heads[1]), min(q_heads[2], q_heads[3]));
                        if (m_pub - head < kUnitQueue) break;
                        if ((spins & 0x3f) == 0) {
                            if (t0 == 0) t0 = global_timer();
                            if (*abort_flag || global_timer() - t0 > kWaitLimitNs) {
                                *abort_flag = 1;
                                if (status_word) *status_word = BSP_ERR_DEVICE_TIMEOUT;
                                alive = false;
                                break;
                            }
                        }
                    }
                    const long long v = (long long)gridDim.x + pend;
                    const int id = (alive && v < n_units) ? (int)v : -1;
                    if (id < 0) closed = true;
                    unit_q[m_pub % kUnitQueue] = id;
                    __threadfence_block();
                    *q_tail = m_pub + 1;
                    ++m_pub;
                    pend_valid = false;
                };
                int n = 0;                 // position in this CTA's unit sequence
                int goff = 0;              // ring entries of the units before this one, mod S
                // this lane's first entry of a unit whose entries start at ring position `off`
                auto first_entry = [&](int b, int off) { return b + (slot - off + S) % S; };
                int u = unit_at(0, true), ub, ue;
                range_of(u, ub, ue);
                int nu = -2, nub = 0, nue = 0;  // the next unit once it is known
                int4 c0 = make_int4(0, 0, 0, 0), c1 = c0, n0 = c0, n1 = c0;
                bool have = false;         // (c0, c1) is the record of this lane's next entry
                uint32_t uses = 0;         // how often this lane's stage has been filled
                while (u >= 0 && alive) {
                    auto peek_next = [&]() {
                        if (nu == -2) {
                            nu = unit_at(n + 1, false);
                            if (nu != -2) range_of(nu, nub, nue);
                        }
                    };
                    peek_next();
                    const int ngoff = (goff + (ue - ub)) % S;
                    for (int e = first_entry(ub, goff); e < ue && alive; e += S) {
                        if (!have) load_rec(e, c0, c1);
                        // fetch this lane's next record now: later in this unit, or its first in the next
                        const int ne = e + S;
                        bool nhave = false;
                        if (ne < ue) {
                            load_rec(ne, n0, n1);
                            nhave = true;
                        } else {
                            peek_next();
                            if (nu >= 0 && first_entry(nub, ngoff) < nue) {
                                load_rec(first_entry(nub, ngoff), n0, n1);
                                nhave = true;
                            }
                        }
                        const int kc = e % KC;
                        int ia = c0.x;
                        int ib[4] = {c0.y, c0.z, c0.w, c1.x};
                        const uint32_t ctrl = (uint32_t)c1.y;
                        const uint32_t present = ctrl & 0xFu;
                        bool bad = ia < 0 || ia >= n_a;
#pragma unroll
                        for (int q = 0; q < G; ++q)
                            if ((present >> q) & 1u) bad |= ib[q] < 0 || ib[q] >= n_b;
                        if (bad) {
                            if (status_word) *status_word = BSP_ERR_DEVICE_RANGE;
                            ia = 0;
#pragma unroll
                            for (int q = 0; q < 4; ++q) ib[q] = 0;
                        }
                        const uint32_t phase = uses & 1u;
                        const uint32_t ebar = empty_bar + 8 * slot, fbar = full_bar + 8 * slot;
                        const uint32_t sa = data + slot * L::kStageBytes;
                        const uint32_t sb = sa + L::kChunkBytes;
                        unsigned long long t0 = 0;
                        for (uint32_t spins = 1;; ++spins) {
                            if (mbar_try_wait(ebar, phase ^ 1u)) {
                                // first-touch flags count for the step's first chunk only; the panel ends
                                // with the step's last chunk
                                ctrl_slot[slot] = (ctrl & (kc == 0 ? ~0u : ~0xF0u)) & (kc == KC - 1 ? ~0u : ~kCtrlLast);
                                armed[slot] = (int)phase;
                                mbar_arrive_expect_tx(fbar, (1 + __popc(present)) * L::kChunkBytes);
                                if (A_MN) {
#pragma unroll
                                    for (int h = 0; h < H; ++h)
                                        tma_load_2d(sa + h * ATOM, &map_a, h * KE, ia * BS + kc * KE, fbar);
                                } else {
                                    tma_load_2d(sa, &map_a, kc * KE, ia * BS, fbar);
                                }
#pragma unroll
                                for (int q = 0; q < G; ++q) {
                                    if ((present >> q) & 1u) {
                                        if (B_MN) {
#pragma unroll
                                            for (int h = 0; h < H; ++h)
                                                tma_load_2d(sb + (q * H + h) * ATOM, &map_b, h * KE, ib[q] * BS + kc * KE, fbar);
                                        } else {
                                            tma_load_2d(sb + q * L::kChunkBytes, &map_b, kc * KE, ib[q] * BS, fbar);
                                        }
                                    }
                                }
                                ++uses;
                                break;
                            }
                            if ((spins & 0xff) == 0) {
                                if (t0 == 0) t0 = global_timer();
                                if (*abort_flag || global_timer() - t0 > kWaitLimitNs) {
                                    *abort_flag = 1;
                                    if (status_word) *status_word = BSP_ERR_DEVICE_TIMEOUT;
                                    alive = false;
                                    break;
                                }
                            }
                        }
                        if (scheduler && !closed) {
                            if (pend_valid) {
                                if (++pend_age >= 2) publish();
                            } else if (m_pub <= n + 2) {
                                draw();
                            }
                        }
                        have = nhave;
                        c0 = n0;
                        c1 = n1;
                    }
                    if (scheduler && !closed && m_pub <= n + 1) {
                        // the next unit has to be known now
                        if (!pend_valid) draw();
                        publish();
                    }
                    if (!alive) break;
                    if (nu == -2) {
                        nu = unit_at(n + 1, true);
                        range_of(nu, nub, nue);
                    }
                    u = nu;
                    ub = nub;
                    ue = nue;
                    goff = ngoff;
                    nu = -2;
                    ++n;
                }
            }
        } else if (warp == S) {
            // ---------------- MMA issuer ----------------
            // The whole warp runs this loop converged and one elected lane issues each MMA / commit:
            // stage, descriptor and accumulator arithmetic is then warp-uniform (uniform registers)
            // instead of one diverged lane's, which shortens the issue path measurably.
            {
                int grp = 0, stage = 0;     // ring stages are used round-robin across unit boundaries
                uint32_t stage_parity = 0;  // bit s = parity of the next fill of stage s
                uint32_t grp_phase = 0;
                bool new_panel = true, alive = true;
                auto entries_of = [&](int uu) { return uu >= 0 ? (unit_step[uu + 1] - unit_step[uu]) * KC : 0; };
                int n = 0;  // position in this CTA's unit sequence
                int u = unit_at(0, true);
                int n_entries = entries_of(u);
                while (u >= 0 && alive) {
                    // the next unit's size is fetched early when its number is already known
                    int nu = unit_at(n + 1, false);
                    int next_entries = entries_of(nu);
                    for (int e = 0; e < n_entries; ++e) {
                        if (new_panel) {
                            if (!mbar_wait(tempty_bar + 8 * grp, grp_phase ^ 1u, abort_flag, status_word)) { alive = false; break; }
                        }
                        if (!mbar_wait(full_bar + 8 * stage, (stage_parity >> stage) & 1u, abort_flag, status_word)) { alive = false; break; }
                        stage_parity ^= 1u << stage;
                        tc_fence_after();
                        const uint32_t ctrl = ctrl_slot[stage];
                        const uint32_t present = ctrl & 0xFu, first = (ctrl >> 4) & 0xFu;
                        const uint32_t sa = data + stage * L::kStageBytes;
                        const uint32_t sb = sa + L::kChunkBytes;
                        const uint32_t d0 = tmem_base + grp * (G * BS);
                        if constexpr (G == 1) {
                            // a step is one (A, B) pair
                            const uint32_t idesc = idesc_no_n | ((uint32_t)(BS >> 3) << 17);
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                tc_mma_elect<T>(d0, chunk_desc<T, A_MN>(sa, kk), chunk_desc<T, B_MN>(sb, kk), idesc,
                                                 ((first & 1u) && kk == 0) ? 0u : 1u);
                            }
                        } else {
                            // one MMA chain per run of present columns with equal "first" status
                            int q = 0;
                            while (q < G) {
                                if (!((present >> q) & 1u)) { ++q; continue; }
                                const int q0 = q;
                                const uint32_t f = (first >> q) & 1u;  // zero on later chunks of a step
                                ++q;
                                while (q < G && ((present >> q) & 1u) && ((first >> q) & 1u) == f) ++q;
                                const uint32_t n = (uint32_t)(q - q0) * BS;
                                const uint32_t idesc = idesc_no_n | ((n >> 3) << 17);
                                // the run's first B sub-tile: K-major blocks follow each other row after
                                // row, MN-major blocks are bs/64 atoms of 8 KiB each
                                const uint32_t sbq = sb + (B_MN ? q0 * H * ATOM : q0 * L::kChunkBytes);
#pragma unroll
                                for (int kk = 0; kk < 4; ++kk) {
                                    tc_mma_elect<T>(d0 + q0 * BS, chunk_desc<T, A_MN>(sa, kk),
                                                    chunk_desc<T, B_MN>(sbq, kk), idesc, (f && kk == 0) ? 0u : 1u);
                                }
                            }
                        }
                        tc_commit_elect(empty_bar + 8 * stage);
                        new_panel = false;
                        if (ctrl & kCtrlLast) {
                            tc_commit_elect(tfull_bar + 8 * grp);
                            new_panel = true;
                            if (++grp == NG) { grp = 0; grp_phase ^= 1u; }
                        }
                        if (++stage == S) stage = 0;
                    }
                    if (!alive) break;
                    if (nu == -2) {
                        nu = unit_at(n + 1, true);
                        next_entries = entries_of(nu);
                    }
                    u = nu;
                    n_entries = next_entries;
                    ++n;
                }
                // every MMA issued so far has to complete before tensor memory may be freed; this wait has
                // its own limit and does not give up early because another role has aborted
                tc_commit_elect(drain_bar);
                mbar_wait_slow(drain_bar, 0, abort_flag, status_word, kWaitLimitNs, false);
            }
        } else {
            // ---------------- epilogue ----------------
            const int wq = warp & 3;  // tensor-memory subpartition of this warp
            constexpr int ROWS_PER_WARP = BS / 4;
            const bool row_valid = lane < ROWS_PER_WARP;
            const int row = wq * ROWS_PER_WARP + lane;
            int grp = 0;
            uint32_t grp_phase = 0;
            bool alive = true;
            // the bias row of output block p (nullptr without a bias): bias[column block * BS ...]
            auto bias_of = [&](int p) -> const T* {
                if constexpr (!BIAS) return nullptr;
                return bias + out_lut[(int64_t)p * 3 + 2] * BS;
            };
            // a block nothing was accumulated into: zeros, or the bias row repeated; in softmax mode its
            // scores are all zero, so exp(s - maximum) = 1 everywhere, maximum 0, sum BS
            auto zero_quarter = [&](T* o, const T* brow, int p) {
                uint4* dst = reinterpret_cast<uint4*>(o + (int64_t)wq * ROWS_PER_WARP * BS);
                constexpr int VECS = ROWS_PER_WARP * BS * (int)sizeof(T) / 16, ROW_VECS = BS * (int)sizeof(T) / 16;
                if (BIAS && brow) {
                    const uint4* bv = reinterpret_cast<const uint4*>(brow);
                    for (int i = lane; i < VECS; i += 32) dst[i] = __ldg(bv + i % ROW_VECS);
                } else if (SOFTMAX) {
                    uint32_t one;
                    if constexpr (sizeof(T) == 4) one = __float_as_uint(1.0f);
                    else one = pack2<T>(1.0f, 1.0f);
                    for (int i = lane; i < VECS; i += 32) dst[i] = make_uint4(one, one, one, one);
                    if (row_valid) stats[(int64_t)p * BS + row] = make_float2(0.f, (float)BS);
                } else {
                    for (int i = lane; i < VECS; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
                }
            };
            // A lane's panel of a batch of 32: (first block, blocks, steps, touched mask).
            auto load_meta = [&](int pi, int pend) -> int4 {
                int4 r = make_int4(0, 0, 0, 0);
                if (pi < pend) {
                    r.x = panel_first[pi];
                    r.y = panel_first[pi + 1] - r.x;
                    r.z = step_off[pi + 1] - step_off[pi];
                    r.w = touched[pi];
                }
                return r;
            };
            // The panel range of the next unit and the panel records of its first batch are fetched
            // while the current unit is being written, so that a unit boundary costs no memory round trip.
            int n = 0;  // position in this CTA's unit sequence
            int u = unit_at(0, true);
            int pn_begin = 0, pn_end = 0;
            if (u >= 0) {
                pn_begin = unit_panel[u];
                pn_end = unit_panel[u + 1];
            }
            int4 meta = load_meta(pn_begin + lane, pn_end);
            bool meta_ok = true;
            while (u >= 0 && alive) {
                int nu = unit_at(n + 1, false), npb = 0, npe = 0;
                if (nu >= 0) {
                    npb = unit_panel[nu];
                    npe = unit_panel[nu + 1];
                }
                int4 nmeta = make_int4(0, 0, 0, 0);
                bool nmeta_ok = false;
                for (int w0 = pn_begin; w0 < pn_end && alive; w0 += 32) {
                    if (!meta_ok) meta = load_meta(w0 + lane, pn_end);
                    meta_ok = false;
                    const int my_first = meta.x, my_g = meta.y, my_steps = meta.z, my_touched = meta.w;
                    const int m = min(32, pn_end - w0);
                    for (int j = 0; j < m && alive; ++j) {
                        if (j == m - 1 && w0 + 32 >= pn_end && nu >= 0) {  // the unit's last panel
                            nmeta = load_meta(npb + lane, npe);
                            nmeta_ok = true;
                        }
                        const int first = __shfl_sync(0xffffffffu, my_first, j);
                        const int g = __shfl_sync(0xffffffffu, my_g, j);
                        const int nsteps = __shfl_sync(0xffffffffu, my_steps, j);
                        const int tmask = __shfl_sync(0xffffffffu, my_touched, j);
                        if (nsteps == 0) {
                            for (int q = 0; q < g; ++q)
                                zero_quarter(out + (int64_t)(first + q) * BS * BS, bias_of(first + q), first + q);
                            continue;
                        }
                        if (!mbar_wait(tfull_bar + 8 * grp, grp_phase, abort_flag, status_word)) alive = false;
                        alive = __all_sync(0xffffffffu, alive);
                        if (!alive) break;
                        tc_fence_after();
                        // The accumulator group goes back to the MMA warp as soon as this warp's last read of
                        // it has landed in registers; conversion, exchange and stores follow after that.
                        bool released = false;
                        auto release_group = [&]() {
                            if (!released) {
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(tempty_bar + 8 * grp);
                                released = true;
                            }
                        };
                        const int touched_here = tmask & ((1 << g) - 1);
                        const int last_q = touched_here ? 31 - __clz(touched_here) : -1;  // last block that holds sums
                        const uint32_t tgroup = tmem_base + grp * (G * BS) + ((uint32_t)(wq * 32) << 16);
                        for (int q = 0; q < g; ++q) {
                            T* o = out + (int64_t)(first + q) * BS * BS;
                            const T* brow = bias_of(first + q);
                            if (!((tmask >> q) & 1)) {
                                zero_quarter(o, brow, first + q);
                                continue;
                            }
                            const uint32_t taddr = tgroup + q * BS;
                            if constexpr (BS == 64) {
                                // M = 64: the warp's 16 rows x 64 columns in one load; all 32 lanes get data
                                uint32_t v[32];
                                tc_ld16x64(taddr, v);
                                tc_wait_ld();
                                if (q == last_q) release_group();
                                const int qd = lane & 3;
                                const int r0 = wq * 16 + (lane >> 2);  // and r0 + 8
                                if (BIAS && brow) {
#pragma unroll
                                    for (int gq = 0; gq < 8; ++gq) {
                                        const float b0 = (float)__ldg(brow + 8 * gq + 2 * qd);
                                        const float b1 = (float)__ldg(brow + 8 * gq + 2 * qd + 1);
                                        v[4 * gq] = __float_as_uint(__uint_as_float(v[4 * gq]) + b0);
                                        v[4 * gq + 1] = __float_as_uint(__uint_as_float(v[4 * gq + 1]) + b1);
                                        v[4 * gq + 2] = __float_as_uint(__uint_as_float(v[4 * gq + 2]) + b0);
                                        v[4 * gq + 3] = __float_as_uint(__uint_as_float(v[4 * gq + 3]) + b1);
                                    }
                                }
                                if constexpr (SOFTMAX) {
                                    // rows r0 (v[4g], v[4g+1]) and r0 + 8 (v[4g+2], v[4g+3]); a row's 64 columns
                                    // are spread over the four threads of a quad
                                    float ma = -FLT_MAX, mb = -FLT_MAX;
#pragma unroll
                                    for (int gq = 0; gq < 8; ++gq) {
#pragma unroll
                                        for (int e = 0; e < 4; ++e) v[4 * gq + e] = __float_as_uint(__uint_as_float(v[4 * gq + e]) * scale);
                                        ma = fmaxf(ma, fmaxf(__uint_as_float(v[4 * gq]), __uint_as_float(v[4 * gq + 1])));
                                        mb = fmaxf(mb, fmaxf(__uint_as_float(v[4 * gq + 2]), __uint_as_float(v[4 * gq + 3])));
                                    }
                                    ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 1));
                                    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
                                    ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 2));
                                    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
                                    float la = 0.f, lb = 0.f;
#pragma unroll
                                    for (int gq = 0; gq < 8; ++gq) {
                                        const float a0 = __expf(__uint_as_float(v[4 * gq]) - ma), a1 = __expf(__uint_as_float(v[4 * gq + 1]) - ma);
                                        const float b0 = __expf(__uint_as_float(v[4 * gq + 2]) - mb), b1 = __expf(__uint_as_float(v[4 * gq + 3]) - mb);
                                        la += a0 + a1;
                                        lb += b0 + b1;
                                        v[4 * gq] = __float_as_uint(a0);
                                        v[4 * gq + 1] = __float_as_uint(a1);
                                        v[4 * gq + 2] = __float_as_uint(b0);
                                        v[4 * gq + 3] = __float_as_uint(b1);
                                    }
                                    la += __shfl_xor_sync(0xffffffffu, la, 1);
                                    lb += __shfl_xor_sync(0xffffffffu, lb, 1);
                                    la += __shfl_xor_sync(0xffffffffu, la, 2);
                                    lb += __shfl_xor_sync(0xffffffffu, lb, 2);
                                    if (qd == 0) {
                                        stats[(int64_t)(first + q) * BS + r0] = make_float2(ma, la);
                                        stats[(int64_t)(first + q) * BS + r0 + 8] = make_float2(mb, lb);
                                    }
                                }
                                T* d0 = o + (int64_t)r0 * BS;
                                T* d1 = d0 + 8 * BS;
                                if constexpr (sizeof(T) == 4) {
                                    // fp32 data: a thread's two adjacent columns are 8 bytes.  Neighbouring lanes
                                    // swap their pieces of two neighbouring column groups (even lanes keep group
                                    // gq, odd lanes group gq + 1), so that every thread stores 16 bytes and a quad
                                    // fills 64 contiguous bytes of each of the two groups' rows.
                                    const bool odd = qd & 1;
#pragma unroll
                                    for (int gq = 0; gq < 8; gq += 2) {
                                        uint32_t ra[4], rb[4];
#pragma unroll
                                        for (int e = 0; e < 2; ++e) {
                                            const uint32_t xa = __shfl_xor_sync(0xffffffffu, odd ? v[4 * gq + e] : v[4 * gq + 4 + e], 1);
                                            const uint32_t xb = __shfl_xor_sync(0xffffffffu, odd ? v[4 * gq + 2 + e] : v[4 * gq + 6 + e], 1);
                                            ra[e] = odd ? xa : v[4 * gq + e];
                                            ra[2 + e] = odd ? v[4 * gq + 4 + e] : xa;
                                            rb[e] = odd ? xb : v[4 * gq + 2 + e];
                                            rb[2 + e] = odd ? v[4 * gq + 6 + e] : xb;
                                        }
                                        const int col = odd ? 8 * (gq + 1) + 2 * (qd - 1) : 8 * gq + 2 * qd;
                                        st_global_16B(d0 + col, ra);
                                        st_global_16B(d1 + col, rb);
                                    }
                                } else {
                                    // 16-bit data: a thread's two columns are one 4-byte word, the four threads
                                    // of a quad hold a row's eight column groups interleaved.  A 4 x 4 exchange
                                    // inside the quad gives every thread 32 contiguous bytes of the row, so that a
                                    // quad writes the row's whole 128-byte line with one 32-byte store per thread.
                                    uint32_t wa[8], wb[8];
#pragma unroll
                                    for (int gq = 0; gq < 8; ++gq) {
                                        wa[gq] = pack2<T>(__uint_as_float(v[4 * gq]), __uint_as_float(v[4 * gq + 1]));
                                        wb[gq] = pack2<T>(__uint_as_float(v[4 * gq + 2]), __uint_as_float(v[4 * gq + 3]));
                                    }
                                    quad_gather8(wa, lane);
                                    quad_gather8(wb, lane);
                                    uint32_t oa[8], ob[8];
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        constexpr int kSlot[8] = {0, 2, 4, 6, 1, 3, 5, 7};  // slot holding output word j
                                        oa[j] = wa[kSlot[j]];
                                        ob[j] = wb[kSlot[j]];
                                    }
                                    st_global_32B(d0 + 16 * qd, oa);
                                    st_global_32B(d1 + 16 * qd, ob);
                                }
                            } else if constexpr (sizeof(T) == 2) {
                                // 16-bit data, lane = row: 64 columns (two loads) are 128 bytes of a row.  An 8 x 8
                                // exchange of 16-byte chunks among the 8 lanes of a group leaves every lane with
                                // the same chunk of the group's 8 rows, so that 8 neighbouring lanes store one
                                // row's whole 128-byte line per instruction.
                                T* obase = o + (int64_t)(wq * 32 + (lane & ~7)) * BS + (lane & 7) * 8;
                                float rmax = -FLT_MAX, rsum = 0.f;  // softmax mode: this lane's row
                                if constexpr (SOFTMAX) rmax = row_max_scaled(taddr, scale);
#pragma unroll
                                for (int half = 0; half < 2; ++half) {
                                    uint32_t v[64];
                                    tc_ld32(taddr + half * 64, v);
                                    tc_ld32(taddr + half * 64 + 32, v + 32);
                                    tc_wait_ld();
                                    if (q == last_q && half == 1) release_group();
                                    if constexpr (SOFTMAX) {
#pragma unroll
                                        for (int e = 0; e < 64; ++e) {
                                            const float ex = __expf(__uint_as_float(v[e]) * scale - rmax);
                                            rsum += ex;
                                            v[e] = __float_as_uint(ex);
                                        }
                                    }
                                    if (BIAS && brow) {
                                        const uint4* bv = reinterpret_cast<const uint4*>(brow + half * 64);
#pragma unroll
                                        for (int i = 0; i < 8; ++i) {
                                            const uint4 b4 = __ldg(bv + i);
                                            const T* be = reinterpret_cast<const T*>(&b4);
#pragma unroll
                                            for (int e = 0; e < 8; ++e)
                                                v[8 * i + e] = __float_as_uint(__uint_as_float(v[8 * i + e]) + (float)be[e]);
                                        }
                                    }
                                    uint32_t w[32];
#pragma unroll
                                    for (int e = 0; e < 32; ++e)
                                        w[e] = pack2<T>(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
                                    octet_gather_chunks(w, lane);
#pragma unroll
                                    for (int i = 0; i < 8; ++i)
                                        st_global_16B(obase + (int64_t)i * BS + half * 64, w + 4 * i);
                                }
                                if constexpr (SOFTMAX) stats[(int64_t)(first + q) * BS + row] = make_float2(rmax, rsum);
                            } else {
                            float rmax = -FLT_MAX, rsum = 0.f;  // softmax mode: this lane's row
                            if constexpr (SOFTMAX && BS == 128) rmax = row_max_scaled(taddr, scale);
#pragma unroll
                            for (int c0 = 0; c0 < BS; c0 += 32) {
                                uint32_t v[32];
                                tc_ld32(taddr + c0, v);
                                tc_wait_ld();
                                if (q == last_q && c0 == BS - 32) release_group();
                                if (BIAS && brow) {
                                    // every lane adds the same 32 bias values (broadcast loads)
                                    constexpr int EPV = 16 / (int)sizeof(T);  // elements per 16-byte load
                                    const uint4* bv = reinterpret_cast<const uint4*>(brow + c0);
#pragma unroll
                                    for (int i = 0; i < 32 / EPV; ++i) {
                                        const uint4 b4 = __ldg(bv + i);
                                        const T* be = reinterpret_cast<const T*>(&b4);
#pragma unroll
                                        for (int e = 0; e < EPV; ++e)
                                            v[EPV * i + e] = __float_as_uint(__uint_as_float(v[EPV * i + e]) + (float)be[e]);
                                    }
                                }
                                if constexpr (SOFTMAX) {
#pragma unroll
                                    for (int e = 0; e < 32; ++e) {
                                        const float ex = __expf(__uint_as_float(v[e]) * scale - rmax);
                                        rsum += ex;
                                        v[e] = __float_as_uint(ex);
                                    }
                                }
                                {
                                    // (fp32 data, block size 128.)  lane = row; 32 fp32 columns are one 128-byte line of the row.  The same
                                    // 8 x 8 exchange of 16-byte chunks as for 16-bit data: afterwards 8
                                    // neighbouring lanes store one row's whole line per instruction.
                                    octet_gather_chunks(v, lane);
                                    T* obase = o + (int64_t)(wq * 32 + (lane & ~7)) * BS + c0 + (lane & 7) * 4;
#pragma unroll
                                    for (int i = 0; i < 8; ++i) st_global_16B(obase + (int64_t)i * BS, v + 4 * i);
                                }
                            }
                            if constexpr (SOFTMAX) {
                                if (row_valid) stats[(int64_t)(first + q) * BS + row] = make_float2(rmax, rsum);
                            }
                            }
                        }
                        release_group();  // a panel whose steps touched none of its blocks
                        if (++grp == NG) { grp = 0; grp_phase ^= 1u; }
                    }
                }
                // this warp is done with position n: its queue slot may be reused
                __syncwarp();
                if (lane == 0) q_heads[wq] = n + 1;
                if (!alive) break;
                if (nu == -2) {
                    nu = unit_at(n + 1, true);
                    if (nu >= 0) {
                        npb = unit_panel[nu];
                        npe = unit_panel[nu + 1];
                    }
                }
                if (nu >= 0 && !nmeta_ok) {
                    nmeta = load_meta(npb + lane, npe);
                    nmeta_ok = true;
                }
                u = nu;
                pn_begin = npb;
                pn_end = npe;
                meta = nmeta;
                meta_ok = nmeta_ok;
                ++n;
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            const int ph = armed[s];
            if (ph >= 0) {
                const unsigned long long t0 = global_timer();
                while (!mbar_try_wait(full_bar + 8 * s, (uint32_t)ph)) {
                    if (global_timer() - t0 > kWaitLimitNs) break;
                }
            }
        }
    }
    __syncthreads();
    if (warp == S) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    // the last CTA to finish puts the scheduling counters back to zero for the next launch
    if (dyn && threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(sched + 1, 1) == (int)gridDim.x - 1) {
            sched[0] = 0;
            sched[1] = 0;
            __threadfence();
        }
    }
}

template <typename T, int BS, int OP, int G, int EPI>
int launch_cfg(const CUtensorMap& ma, const CUtensorMap& mb, int64_t n_a, int64_t n_b, void* out,
               const void* bias, const int64_t* out_lut, float scale, float* stats, const int32_t* panel_first, const int32_t* step_off, const int32_t* steps,
               const int32_t* touched, const int32_t* unit_panel, const int32_t* unit_step, int32_t n_units,
               int32_t* sched, int dtype, int32_t* status_word, cudaStream_t stream) {
    auto kern = matmul_umma_kernel<T, BS, OP, G, EPI>;
    constexpr int smem = PSmem<BS, G>::kTotal;
    // the shared-memory opt-in is a per-device property of this instantiation: set it once per device
    static std::atomic<uint64_t> opted_in{0};
    int dev = 0;
    BSP_CUDA_TRY(cudaGetDevice(&dev));
    const uint64_t dev_bit = dev >= 0 && dev < 64 ? (1ull << dev) : 0;
    if (!(opted_in.load(std::memory_order_acquire) & dev_bit)) {
        BSP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        opted_in.fetch_or(dev_bit, std::memory_order_release);
    }
    const uint32_t idesc_no_n = make_idesc(dtype, BS, OP) & ~(0x3Fu << 17);
    int ctas = num_sms() * PCfg<BS, G>::kCtasPerSm;
    if (ctas > n_units) ctas = n_units;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3((unsigned)PCfg<BS, G>::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see griddepcontrol in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BSP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ma, mb, n_a, n_b, (T*)out, (const T*)bias, out_lut, scale,
                                    reinterpret_cast<float2*>(stats), panel_first, step_off,
                                    steps, touched, unit_panel, unit_step, (int)n_units, idesc_no_n, sched, status_word));
    return BSP_OK;
}

#define BSP_LAUNCH_ARGS ma, mb, n_a, n_b, out, bias, out_lut, scale, stats, panel_first, step_off, steps, touched, unit_panel, unit_step, n_units, sched, dtype, status_word, stream

template <typename T, int BS, int G>
int launch_op(int op, const CUtensorMap& ma, const CUtensorMap& mb, int64_t n_a, int64_t n_b, void* out,
              const void* bias, const int64_t* out_lut, float scale, float* stats, const int32_t* panel_first, const int32_t* step_off, const int32_t* steps, const int32_t* touched,
              const int32_t* unit_panel, const int32_t* unit_step, int32_t n_units, int32_t* sched, int dtype,
              int32_t* status_word, cudaStream_t stream) {
    switch (op) {
        // a bias or the softmax epilogue goes with the forward product only
        case BSP_OP_NN:
            if (bias && stats) return BSP_ERR_UNSUPPORTED;
            if (stats) return launch_cfg<T, BS, BSP_OP_NN, G, kEpiSoftmax>(BSP_LAUNCH_ARGS);
            return bias ? launch_cfg<T, BS, BSP_OP_NN, G, kEpiBias>(BSP_LAUNCH_ARGS)
                        : launch_cfg<T, BS, BSP_OP_NN, G, kEpiPlain>(BSP_LAUNCH_ARGS);
        case BSP_OP_NT:
            return (bias || stats) ? BSP_ERR_UNSUPPORTED : launch_cfg<T, BS, BSP_OP_NT, G, kEpiPlain>(BSP_LAUNCH_ARGS);
        case BSP_OP_TN:
            return (bias || stats) ? BSP_ERR_UNSUPPORTED : launch_cfg<T, BS, BSP_OP_TN, G, kEpiPlain>(BSP_LAUNCH_ARGS);
        default: return BSP_ERR_INVALID_ARG;
    }
}

template <typename T>
int launch_shape(int bs, int width, int op, const CUtensorMap& ma, const CUtensorMap& mb, int64_t n_a, int64_t n_b,
                 void* out, const void* bias, const int64_t* out_lut, float scale, float* stats,
                 const int32_t* panel_first,
                 const int32_t* step_off, const int32_t* steps,
                 const int32_t* touched, const int32_t* unit_panel, const int32_t* unit_step, int32_t n_units,
                 int32_t* sched, int dtype, int32_t* status_word, cudaStream_t stream) {
    if (bs == 64 && width == 1) return launch_op<T, 64, 1>(op, BSP_LAUNCH_ARGS);
    if (bs == 64 && width == 2) return launch_op<T, 64, 2>(op, BSP_LAUNCH_ARGS);
    if (bs == 128 && width == 1) return launch_op<T, 128, 1>(op, BSP_LAUNCH_ARGS);
    if (bs == 128 && width == 2) return launch_op<T, 128, 2>(op, BSP_LAUNCH_ARGS);
    return BSP_ERR_UNSUPPORTED;
}

// Self test of the bounded wait every role of the matmul kernel relies on: one thread waits on
// an mbarrier nothing will ever arrive on, with a short limit, and must come back with
// BSP_ERR_DEVICE_TIMEOUT in the status word instead of hanging.
__global__ void wait_limit_selftest_kernel(unsigned long long limit_ns, int32_t* status_word) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_addr(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_wait_slow(smem_addr(&bar), 0, &abort_flag, status_word, limit_ns);
    }
}

}  // namespace


bool umma_applicable(int dtype, int bs) {
    return (dtype == BSP_F16 || dtype == BSP_BF16 || dtype == BSP_F32) && (bs == 64 || bs == 128);
}

}  // namespace bsp

using namespace bsp;

extern "C" int bsp_selftest_wait_limit(uint32_t limit_us, int32_t* status_word, void* stream_) {
    if (!status_word || limit_us == 0 || limit_us > 100000) return BSP_ERR_INVALID_ARG;  // at most 0.1 s
    wait_limit_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream_>>>((unsigned long long)limit_us * 1000ull, status_word);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

extern "C" int bsp_umma_max_width(int dtype, int bs) {
    return umma_applicable(dtype, bs) ? 2 : 0;
}

extern "C" int bsp_umma_num_ctas(int dtype, int bs, int width) {
    if (!umma_applicable(dtype, bs) || (width != 1 && width != 2)) return 0;
    const int per_sm = bs == 64 ? (width == 1 ? PCfg<64, 1>::kCtasPerSm : PCfg<64, 2>::kCtasPerSm)
                                : (width == 1 ? PCfg<128, 1>::kCtasPerSm : PCfg<128, 2>::kCtasPerSm);
    return umma::num_sms() * per_sm;
}

static int matmul_umma_common(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out, int64_t n_out,
                              const void* bias, const int64_t* out_lut, float scale, float* stats,
                              const int32_t* panel_first, int64_t n_panels, const int32_t* step_off,
                              const int32_t* steps, const int32_t* touched, const int32_t* unit_panel,
                              const int32_t* unit_step, int32_t n_units, int32_t* sched, int width, int bs,
                              int dtype, int op, int32_t* status_word, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_a < 1 || n_b < 1 || n_out < 0 || n_panels < 0) return BSP_ERR_INVALID_ARG;
    if (!umma_applicable(dtype, bs) || (width != 1 && width != 2)) return BSP_ERR_UNSUPPORTED;
    if (op != BSP_OP_NN && op != BSP_OP_NT && op != BSP_OP_TN) return BSP_ERR_INVALID_ARG;
    if (n_out == 0 || n_panels == 0) return BSP_OK;
    if (!a || !b || !out || !panel_first || !step_off || !steps || !touched || !unit_panel || !unit_step ||
        n_units < 1)
        return BSP_ERR_INVALID_ARG;
    // Block rows are the second coordinate of the operands' 2-D tensor maps (32-bit).  At 8 KiB per
    // 64-block of 16-bit data the limit is 33.5 million blocks = 275 GB per operand, beyond the device.
    if (n_a * bs > 0x7fffffffLL || n_b * bs > 0x7fffffffLL || n_out > 0x7fffffffLL) return BSP_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 31) || (reinterpret_cast<uintptr_t>(steps) & 15))
        return BSP_ERR_INVALID_ARG;
    if (bias && (!out_lut || (reinterpret_cast<uintptr_t>(bias) & 15))) return BSP_ERR_INVALID_ARG;
    if (stats && (reinterpret_cast<uintptr_t>(stats) & 7)) return BSP_ERR_INVALID_ARG;
    CUtensorMap ma, mb;
    // a block read MN-major is fetched 64 rows at a time, one read K-major as bs rows x 64 columns
    int st = umma::make_block_map(&ma, a, n_a, bs, dtype, op == BSP_OP_TN);
    if (st != BSP_OK) return st;
    st = umma::make_block_map(&mb, b, n_b, bs, dtype, op != BSP_OP_NT);
    if (st != BSP_OK) return st;
    if (dtype == BSP_F32) return launch_shape<float>(bs, width, op, BSP_LAUNCH_ARGS);
    if (dtype == BSP_F16) return launch_shape<__half>(bs, width, op, BSP_LAUNCH_ARGS);
    return launch_shape<__nv_bfloat16>(bs, width, op, BSP_LAUNCH_ARGS);
}

extern "C" int bsp_matmul_umma(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out, int64_t n_out,
                               const void* bias, const int64_t* out_lut, const int32_t* panel_first, int64_t n_panels, const int32_t* step_off,
                               const int32_t* steps, const int32_t* touched, const int32_t* unit_panel,
                               const int32_t* unit_step, int32_t n_units, int32_t* sched, int width, int bs,
                               int dtype, int op, int32_t* status_word, void* stream_) {
    return matmul_umma_common(a, n_a, b, n_b, out, n_out, bias, out_lut, 1.0f, nullptr, panel_first, n_panels, step_off,
                              steps, touched, unit_panel, unit_step, n_units, sched, width, bs, dtype, op, status_word,
                              stream_);
}

extern "C" int bsp_matmul_umma_softmax(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                                       int64_t n_out, float* stats, float scale, const int32_t* panel_first,
                                       int64_t n_panels, const int32_t* step_off, const int32_t* steps,
                                       const int32_t* touched, const int32_t* unit_panel, const int32_t* unit_step,
                                       int32_t n_units, int32_t* sched, int width, int bs, int dtype,
                                       int32_t* status_word, void* stream_) {
    if (n_out > 0 && !stats) return BSP_ERR_INVALID_ARG;
    return matmul_umma_common(a, n_a, b, n_b, out, n_out, nullptr, nullptr, scale, stats, panel_first, n_panels,
                              step_off, steps, touched, unit_panel, unit_step, n_units, sched, width, bs, dtype,
                              BSP_OP_NN, status_word, stream_);
}
