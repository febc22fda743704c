// Wide-N variant of the tcgen05 block-sparse matmul: works on panels of up to G output blocks
// of one output row (see plan_panel.cu).  Per step one A block and the step's B blocks are
// staged; the B blocks of neighbouring panel columns lie side by side in shared memory, so a
// run of present columns is multiplied by ONE tcgen05.mma of N = run x bs, and the A block is
// fetched once per step instead of once per (A, B) pair.  With dense B operands (attention
// scores, P*V, sparse x dense) every MMA is N = G*bs wide.
//
// A ring entry is one (step, k-chunk): 64 of the bs contraction indices of the step's blocks,
// so that for bs = 128 the MMAs of the first half can start while the second half is in flight.
// A block read K-major contributes its 64-column half k (bs rows x 128 B); a block read
// MN-major contributes rows [64k, 64k+64) as bs/64 sub-tiles of 64 rows x 128 B.
//
// Roles as in matmul_umma.cu: warp 0 producer (lane l owns ring stage l), warp 1 MMA issuer,
// warps 2-5 epilogue.  An accumulator group holds the G accumulators of a panel in adjacent
// tensor-memory columns.  All waits are bounded; see matmul_umma.cu for the abort protocol.
#include "common.cuh"
#include "umma_common.cuh"

namespace bsp {

using namespace umma;

namespace {

constexpr int kThreads = 192;
constexpr uint32_t kCtrlLast = 0x100u;

#ifndef BSP_PANEL64_G
#define BSP_PANEL64_G 2
#endif
#ifndef BSP_PANEL64_STAGES
#define BSP_PANEL64_STAGES 4
#endif
#ifndef BSP_PANEL64_GROUPS
#define BSP_PANEL64_GROUPS 2
#endif
#ifndef BSP_PANEL64_CTAS
#define BSP_PANEL64_CTAS 2
#endif

template <int BS> struct PCfg;
template <> struct PCfg<64> {
    static constexpr int kG = BSP_PANEL64_G;            // output blocks per panel
    static constexpr int kStages = BSP_PANEL64_STAGES;  // x (1 + G) x 8 KiB
    static constexpr int kGroups = BSP_PANEL64_GROUPS;  // accumulator groups of G x 64 columns
    static constexpr int kCtasPerSm = BSP_PANEL64_CTAS;
};
template <> struct PCfg<128> {
    static constexpr int kG = 2;
    static constexpr int kStages = 4;   // 4 x 48 KiB
    static constexpr int kGroups = 2;   // 2 x 256 columns
    static constexpr int kCtasPerSm = 1;
};

constexpr int tmem_cols_pow2(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

template <int BS>
struct PSmem {
    static constexpr int kG = PCfg<BS>::kG;
    static constexpr int kChunkBytes = BS * 128;           // one block's share of a ring entry: bs x 64 elements
    static constexpr int kStageBytes = (1 + kG) * kChunkBytes;
    static constexpr int kDataBytes = PCfg<BS>::kStages * kStageBytes;
    static constexpr int kBarBytes = (2 * PCfg<BS>::kStages + 2 * PCfg<BS>::kGroups + 1) * 8;
    static constexpr int kMiscBytes = (2 * PCfg<BS>::kStages + 2) * 4;
    static constexpr int kTotal = kDataBytes + kBarBytes + kMiscBytes + 1024;
};

// Shared-memory matrix descriptors of a ring entry (all 128-byte swizzle, 8-row groups 1024 B
// apart).  K-major: rows are M/N indices, 16 contraction elements = 32 bytes along the row.
// MN-major: rows are contraction indices (16 rows = 2048 B per MMA), the M/N extent is cut
// into 64-wide atoms of 64 rows x 128 B = 8 KiB, `LBO` apart.
template <int BS, bool MN_MAJOR>
__device__ __forceinline__ uint64_t chunk_desc(uint32_t base, int kk) {
    if (MN_MAJOR) return make_smem_desc(base + kk * 2048, 8192, 1024);
    return make_smem_desc(base + kk * 32, 16, 1024);
}

template <typename T, int BS, int OP>
__global__ void __launch_bounds__(kThreads, PCfg<BS>::kCtasPerSm)
matmul_umma_panel_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         int64_t n_a, int64_t n_b, T* __restrict__ out,
                         const int32_t* __restrict__ panel_first, const int32_t* __restrict__ step_off,
                         const int32_t* __restrict__ steps, const int32_t* __restrict__ touched,
                         const int32_t* __restrict__ chunk_begin, uint32_t idesc_no_n,
                         int32_t* __restrict__ status_word) {
    using C = PCfg<BS>;
    using L = PSmem<BS>;
    constexpr int S = C::kStages, NG = C::kGroups, G = C::kG, H = BS / 64, KC = BS / 64;
    constexpr bool A_MN = (OP == BSP_OP_TN);
    constexpr bool B_MN = (OP != BSP_OP_NT);
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

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pn_begin = chunk_begin[blockIdx.x], pn_end = chunk_begin[blockIdx.x + 1];

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
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_addr((const void*)tmem_base_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (pn_begin < pn_end) {
        const int st_begin = step_off[pn_begin], st_end = step_off[pn_end];

        if (warp == 0) {
            // ---------------- producer: lane l owns ring stage l ----------------
            // ring entry e = (step, k-chunk) = (e / KC, e % KC), counted from the range's first step
            const int4* recs = reinterpret_cast<const int4*>(steps);
            const int n_entries = (st_end - st_begin) * KC;
            uint32_t phase = 0;
            auto load_rec = [&](int e0, int4& r0, int4& r1) {
                const int e = e0 + lane;
                if (lane < S && e < n_entries) {
                    const int64_t i = st_begin + e / KC;
                    r0 = recs[2 * i];
                    r1 = recs[2 * i + 1];
                } else {
                    r0 = make_int4(0, -1, -1, -1);
                    r1 = make_int4(-1, 0, 0, 0);
                }
            };
            int4 c0, c1, n0, n1;
            load_rec(0, c0, c1);
            bool alive = true;
            for (int e0 = 0; e0 < n_entries && alive; e0 += S) {
                load_rec(e0 + S, n0, n1);
                if (lane < S && e0 + lane < n_entries) {
                    const int kc = (e0 + lane) % KC;
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
                    const uint32_t ebar = empty_bar + 8 * lane, fbar = full_bar + 8 * lane;
                    const uint32_t sa = data + lane * L::kStageBytes;
                    const uint32_t sb = sa + L::kChunkBytes;
                    unsigned long long t0 = 0;
                    for (uint32_t spins = 1;; ++spins) {
                        if (mbar_try_wait(ebar, phase ^ 1u)) {
                            // first-touch flags count for the step's first chunk only; the panel ends
                            // with the step's last chunk
                            ctrl_slot[lane] = (ctrl & (kc == 0 ? ~0u : ~0xF0u)) & (kc == KC - 1 ? ~0u : ~kCtrlLast);
                            armed[lane] = (int)phase;
                            mbar_arrive_expect_tx(fbar, (1 + __popc(present)) * L::kChunkBytes);
                            if (A_MN) {
#pragma unroll
                                for (int h = 0; h < H; ++h)
                                    tma_load_2d(sa + h * 8192, &map_a, h * 64, ia * BS + kc * 64, fbar);
                            } else {
                                tma_load_2d(sa, &map_a, kc * 64, ia * BS, fbar);
                            }
#pragma unroll
                            for (int q = 0; q < G; ++q) {
                                if ((present >> q) & 1u) {
                                    if (B_MN) {
#pragma unroll
                                        for (int h = 0; h < H; ++h)
                                            tma_load_2d(sb + (q * H + h) * 8192, &map_b, h * 64, ib[q] * BS + kc * 64, fbar);
                                    } else {
                                        tma_load_2d(sb + q * L::kChunkBytes, &map_b, kc * 64, ib[q] * BS, fbar);
                                    }
                                }
                            }
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
                }
                alive = __all_sync(0xffffffffu, alive);
                phase ^= 1u;
                c0 = n0;
                c1 = n1;
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                int stage = 0, grp = 0;
                uint32_t phase = 0, grp_phase = 0;
                bool new_panel = true;
                const int n_entries = (st_end - st_begin) * KC;
                for (int e = 0; e < n_entries; ++e) {
                    if (new_panel) {
                        if (!mbar_wait(tempty_bar + 8 * grp, grp_phase ^ 1u, abort_flag, status_word)) break;
                    }
                    if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, status_word)) break;
                    tc_fence_after();
                    const uint32_t ctrl = ctrl_slot[stage];
                    const uint32_t present = ctrl & 0xFu, first = (ctrl >> 4) & 0xFu;
                    const uint32_t sa = data + stage * L::kStageBytes;
                    const uint32_t sb = sa + L::kChunkBytes;
                    const uint32_t d0 = tmem_base + grp * (G * BS);
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
                        // the run's first B sub-tile: K-major blocks follow each other row after row,
                        // MN-major blocks are bs/64 atoms of 8 KiB each
                        const uint32_t sbq = sb + (B_MN ? q0 * H * 8192 : q0 * L::kChunkBytes);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            tc_mma_f16(d0 + q0 * BS, chunk_desc<BS, A_MN>(sa, kk), chunk_desc<BS, B_MN>(sbq, kk), idesc,
                                       (f && kk == 0) ? 0u : 1u);
                        }
                    }
                    tc_commit(empty_bar + 8 * stage);
                    new_panel = false;
                    if (ctrl & kCtrlLast) {
                        tc_commit(tfull_bar + 8 * grp);
                        new_panel = true;
                        if (++grp == NG) { grp = 0; grp_phase ^= 1u; }
                    }
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
                tc_commit(drain_bar);
                mbar_wait(drain_bar, 0, abort_flag, status_word);
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
            auto zero_quarter = [&](T* o) {
                uint4* dst = reinterpret_cast<uint4*>(o + (int64_t)wq * ROWS_PER_WARP * BS);
                constexpr int VECS = ROWS_PER_WARP * BS * 2 / 16;
                for (int i = lane; i < VECS; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
            };
            for (int w0 = pn_begin; w0 < pn_end && alive; w0 += 32) {
                const int pi = w0 + lane;
                int my_first = 0, my_g = 0, my_steps = 0, my_touched = 0;
                if (pi < pn_end) {
                    my_first = panel_first[pi];
                    my_g = panel_first[pi + 1] - my_first;
                    my_steps = step_off[pi + 1] - step_off[pi];
                    my_touched = touched[pi];
                }
                const int m = min(32, pn_end - w0);
                for (int j = 0; j < m && alive; ++j) {
                    const int first = __shfl_sync(0xffffffffu, my_first, j);
                    const int g = __shfl_sync(0xffffffffu, my_g, j);
                    const int nsteps = __shfl_sync(0xffffffffu, my_steps, j);
                    const int tmask = __shfl_sync(0xffffffffu, my_touched, j);
                    if (nsteps == 0) {
                        for (int q = 0; q < g; ++q) zero_quarter(out + (int64_t)(first + q) * BS * BS);
                        continue;
                    }
                    if (!mbar_wait(tfull_bar + 8 * grp, grp_phase, abort_flag, status_word)) alive = false;
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    tc_fence_after();
                    for (int q = 0; q < g; ++q) {
                        T* o = out + (int64_t)(first + q) * BS * BS;
                        if (!((tmask >> q) & 1)) {
                            zero_quarter(o);
                            continue;
                        }
                        const uint32_t taddr = tmem_base + grp * (G * BS) + q * BS + ((uint32_t)(wq * 32) << 16);
#pragma unroll
                        for (int c0 = 0; c0 < BS; c0 += 32) {
                            uint32_t v[32];
                            tc_ld32(taddr + c0, v);
                            tc_wait_ld();
                            if (row_valid) {
                                T* dst = o + (int64_t)row * BS + c0;
#pragma unroll
                                for (int i = 0; i < 2; ++i) {
                                    uint32_t u[8];
#pragma unroll
                                    for (int e = 0; e < 8; ++e)
                                        u[e] = pack2<T>(__uint_as_float(v[16 * i + 2 * e]),
                                                        __uint_as_float(v[16 * i + 2 * e + 1]));
                                    st_global_32B(dst + 16 * i, u);
                                }
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar + 8 * grp);
                    if (++grp == NG) { grp = 0; grp_phase ^= 1u; }
                }
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
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

template <typename T, int BS, int OP>
int launch_cfg(const CUtensorMap& ma, const CUtensorMap& mb, int64_t n_a, int64_t n_b, void* out,
               const int32_t* panel_first, const int32_t* step_off, const int32_t* steps,
               const int32_t* touched, const int32_t* chunk_begin, int32_t n_chunks, int dtype,
               int32_t* status_word, cudaStream_t stream) {
    auto kern = matmul_umma_panel_kernel<T, BS, OP>;
    constexpr int smem = PSmem<BS>::kTotal;
    BSP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const uint32_t idesc_no_n = make_idesc(dtype, BS, OP) & ~(0x3Fu << 17);
    kern<<<n_chunks, kThreads, smem, stream>>>(ma, mb, n_a, n_b, (T*)out, panel_first, step_off, steps, touched,
                                               chunk_begin, idesc_no_n, status_word);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

template <typename T, int BS>
int launch_op(int op, const CUtensorMap& ma, const CUtensorMap& mb, int64_t n_a, int64_t n_b, void* out,
              const int32_t* panel_first, const int32_t* step_off, const int32_t* steps, const int32_t* touched,
              const int32_t* chunk_begin, int32_t n_chunks, int dtype, int32_t* status_word, cudaStream_t stream) {
    switch (op) {
        case BSP_OP_NN: return launch_cfg<T, BS, BSP_OP_NN>(ma, mb, n_a, n_b, out, panel_first, step_off, steps, touched, chunk_begin, n_chunks, dtype, status_word, stream);
        case BSP_OP_NT: return launch_cfg<T, BS, BSP_OP_NT>(ma, mb, n_a, n_b, out, panel_first, step_off, steps, touched, chunk_begin, n_chunks, dtype, status_word, stream);
        case BSP_OP_TN: return launch_cfg<T, BS, BSP_OP_TN>(ma, mb, n_a, n_b, out, panel_first, step_off, steps, touched, chunk_begin, n_chunks, dtype, status_word, stream);
        default: return BSP_ERR_INVALID_ARG;
    }
}

}  // namespace

}  // namespace bsp

using namespace bsp;

extern "C" int bsp_panel_width(int dtype, int bs) {
    if (!umma_applicable(dtype, bs)) return 0;
    return bs == 64 ? PCfg<64>::kG : PCfg<128>::kG;
}

extern "C" int bsp_matmul_panel_num_chunks(int dtype, int bs) {
    if (!umma_applicable(dtype, bs)) return 0;
    return umma::num_sms() * (bs == 64 ? PCfg<64>::kCtasPerSm : PCfg<128>::kCtasPerSm);
}

extern "C" int bsp_matmul_panel(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out, int64_t n_out,
                                const int32_t* panel_first, int64_t n_panels, const int32_t* step_offsets,
                                const int32_t* steps, const int32_t* touched, const int32_t* chunk_begin,
                                int32_t n_chunks, int bs, int dtype, int op, int32_t* status_word, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_a < 1 || n_b < 1 || n_out < 0 || n_panels < 0) return BSP_ERR_INVALID_ARG;
    if (!umma_applicable(dtype, bs)) return BSP_ERR_UNSUPPORTED;
    if (op != BSP_OP_NN && op != BSP_OP_NT && op != BSP_OP_TN) return BSP_ERR_INVALID_ARG;
    if (n_out == 0 || n_panels == 0) return BSP_OK;
    if (!a || !b || !out || !panel_first || !step_offsets || !steps || !touched || !chunk_begin || n_chunks < 1)
        return BSP_ERR_INVALID_ARG;
    if (n_a * bs > 0x7fffffffLL || n_b * bs > 0x7fffffffLL || n_out > 0x7fffffffLL) return BSP_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 31) || (reinterpret_cast<uintptr_t>(steps) & 15))
        return BSP_ERR_INVALID_ARG;
    CUtensorMap ma, mb;
    // a block read MN-major is fetched 64 rows at a time, one read K-major as bs rows x 64 columns
    int st = umma::make_block_map(&ma, a, n_a, bs, dtype, op == BSP_OP_TN ? 64 : bs);
    if (st != BSP_OK) return st;
    st = umma::make_block_map(&mb, b, n_b, bs, dtype, op != BSP_OP_NT ? 64 : bs);
    if (st != BSP_OK) return st;
    if (dtype == BSP_F16) {
        if (bs == 64) return launch_op<__half, 64>(op, ma, mb, n_a, n_b, out, panel_first, step_offsets, steps, touched, chunk_begin, n_chunks, dtype, status_word, stream);
        return launch_op<__half, 128>(op, ma, mb, n_a, n_b, out, panel_first, step_offsets, steps, touched, chunk_begin, n_chunks, dtype, status_word, stream);
    }
    if (bs == 64) return launch_op<__nv_bfloat16, 64>(op, ma, mb, n_a, n_b, out, panel_first, step_offsets, steps, touched, chunk_begin, n_chunks, dtype, status_word, stream);
    return launch_op<__nv_bfloat16, 128>(op, ma, mb, n_a, n_b, out, panel_first, step_offsets, steps, touched, chunk_begin, n_chunks, dtype, status_word, stream);
}
