// Block-sparse matmul on a pair plan with 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory) for 16-bit data and block sizes
// 64 and 128.
//
// One persistent CTA per SM walks a contiguous range of output blocks
// (bsp_plan_schedule).  Roles, by warp:
//   warp 0      producer: streams the range's (a_block, b_block) pairs, and for
//               each pair TMA-loads the two bs x bs operand blocks (128-byte
//               swizzle, global orientation) into the next free ring stage
//   warp 1      MMA issuer: one thread issues bs/16 tcgen05.mma per pair into
//               the current accumulator, releases the stage with
//               tcgen05.commit, and hands a finished accumulator to the
//               epilogue
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator, convert to the
//               output type, write the output block; blocks without pairs are
//               written as zeros without touching tensor memory
// The transposed products of the backward pass (BSP_OP_NT, BSP_OP_TN) use the
// same staged blocks; only the major-ness bits of the shared-memory matrix
// descriptors and of the instruction descriptor change.
//
// Every wait is bounded (about one second); a wait that runs out records
// BSP_ERR_DEVICE_TIMEOUT in the status word, all roles leave their loops,
// outstanding copies and MMAs are drained with bounded waits, tensor memory is
// freed and the kernel returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "umma_common.cuh"

namespace bsp {

using namespace umma;

namespace {

constexpr int kThreads = 192;
constexpr uint32_t kFlagLast = 1u;  // stage holds the last pair of its output block
constexpr int kPairLastBit = 0x40000000;   // set on pairs[2p] when p is the last pair of its block
constexpr int kPairIndexMask = 0x3fffffff;

#ifdef BSP_UMMA_PROFILE
// Debug build only: per-CTA cycle counters (8 per CTA) read back by bsp_debug_read_prof.
__device__ long long g_prof[1024 * 8];
#define PROF_DECL(name) long long name = 0
#define PROF_T0(t) long long t = clock64()
#define PROF_ADD(acc, t) acc += clock64() - t
#define PROF_STORE(i, v) g_prof[blockIdx.x * 8 + (i)] = (v)
#else
#define PROF_DECL(name)
#define PROF_T0(t)
#define PROF_ADD(acc, t)
#define PROF_STORE(i, v)
#endif

template <int BS> struct Cfg;
#ifndef BSP_UMMA64_STAGES
#define BSP_UMMA64_STAGES 4
#endif
#ifndef BSP_UMMA64_CTAS
#define BSP_UMMA64_CTAS 3
#endif
#ifndef BSP_UMMA64_ACCS
#define BSP_UMMA64_ACCS 2
#endif

template <> struct Cfg<64> {
    static constexpr int kStages = BSP_UMMA64_STAGES;  // x 16 KiB
    static constexpr int kAccs = BSP_UMMA64_ACCS;      // x 64 columns
    static constexpr int kTmemCols = 64 * BSP_UMMA64_ACCS;
    static constexpr int kCtasPerSm = BSP_UMMA64_CTAS;
};
template <> struct Cfg<128> {
    static constexpr int kStages = 3;     // 3 x 64 KiB
    static constexpr int kAccs = 4;       // 4 x 128 columns
    static constexpr int kTmemCols = 512;
    static constexpr int kCtasPerSm = 1;
};

template <int BS>
struct SmemLayout {
    static constexpr int kBlockBytes = BS * BS * 2;
    static constexpr int kStageBytes = 2 * kBlockBytes;
    static constexpr int kDataBytes = Cfg<BS>::kStages * kStageBytes;
    // after the data: full[S], empty[S], tmem_full[A], tmem_empty[A], drain (8 B each),
    // flags[S] (4 B), armed[S] (4 B), tmem base (4 B), abort flag (4 B)
    static constexpr int kBarBytes = (2 * Cfg<BS>::kStages + 2 * Cfg<BS>::kAccs + 1) * 8;
    static constexpr int kMiscBytes = (2 * Cfg<BS>::kStages + 2) * 4;
    static constexpr int kTotal = kDataBytes + kBarBytes + kMiscBytes + 1024 /* alignment slack */;
};

// A staged operand block is bs rows of bs 16-bit elements, split into column
// panels of 64 elements (128 B): panel h lives at h * bs * 128 bytes, row r of
// a panel at r * 128, 16-byte chunks XOR-swizzled by (r % 8).
//
// Read K-major (the contraction index runs along the rows' 64-element panels):
//   8-row groups are 1024 B apart (SBO); k-step s (16 elements) starts
//   (s / 4) panels in, (s % 4) * 32 bytes into the 128-byte row.
// Read MN-major (the contraction index runs down the rows):
//   the 64-wide panels are the M/N atoms, bs * 128 bytes apart (LBO); 8-row
//   k-groups are 1024 B apart (SBO); k-step s starts 16 rows = 2048 B further.
template <int BS, bool MN_MAJOR>
__device__ __forceinline__ uint64_t operand_desc(uint32_t base, int kstep) {
    if (MN_MAJOR) return make_smem_desc(base + kstep * 2048, BS * 128, 1024);
    return make_smem_desc(base + (kstep >> 2) * (BS * 128) + (kstep & 3) * 32, 16, 1024);
}

template <typename T, int BS, int OP>
__global__ void __launch_bounds__(kThreads, Cfg<BS>::kCtasPerSm)
matmul_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   int64_t n_a, int64_t n_b, T* __restrict__ out,
                   const int32_t* __restrict__ offsets, const int32_t* __restrict__ pairs,
                   const int32_t* __restrict__ chunk_begin, uint32_t idesc,
                   int32_t* __restrict__ status_word) {
    using C = Cfg<BS>;
    using L = SmemLayout<BS>;
    constexpr int S = C::kStages, A = C::kAccs;
    constexpr bool A_MN = (OP == BSP_OP_TN);   // A block is read transposed
    constexpr bool B_MN = (OP != BSP_OP_NT);   // B block rows are the contraction index
    constexpr int KSTEPS = BS / 16;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t data = (raw + 1023u) & ~1023u;
    unsigned char* data_ptr = smem_raw + (data - raw);
    const uint32_t bars = data + L::kDataBytes;
    const uint32_t full_bar = bars, empty_bar = bars + 8 * S, tfull_bar = bars + 16 * S,
                   tempty_bar = tfull_bar + 8 * A, drain_bar = tempty_bar + 8 * A;
    volatile uint32_t* flags = reinterpret_cast<volatile uint32_t*>(data_ptr + L::kDataBytes + L::kBarBytes);
    volatile int* armed = reinterpret_cast<volatile int*>(flags + S);
    volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(armed + S);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk_begin = chunk_begin[blockIdx.x], blk_end = chunk_begin[blockIdx.x + 1];

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
            armed[s] = -1;
        }
        for (int i = 0; i < A; ++i) {
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
                     ::"r"(smem_addr((const void*)tmem_base_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (blk_begin < blk_end) {
        const int pr_begin = offsets[blk_begin], pr_end = offsets[blk_end];

        if (warp == 0) {
            // ---------------- producer ----------------
            // Pairs are handled in rounds of S: in a round lane l (< S) owns pair p0 + l and ring
            // stage l.  Each lane polls its own stage's "empty" barrier and issues its two block
            // copies as soon as that stage is free, so up to S copies are issued per instruction.
            const int2* pairs2 = reinterpret_cast<const int2*>(pairs);
            uint32_t phase = 0;
            auto load_round = [&](int p0) -> int2 {
                const int i = p0 + lane;
                return (lane < S && i < pr_end) ? pairs2[i] : make_int2(0, 0);
            };
            int2 cur = load_round(pr_begin);
            bool alive = true;
            PROF_DECL(w_empty);
            PROF_T0(t_start);
            for (int p0 = pr_begin; p0 < pr_end && alive; p0 += S) {
                const int2 nxt = load_round(p0 + S);
                if (lane < S && p0 + lane < pr_end) {
                    int ia = cur.x & kPairIndexMask, ib = cur.y;
                    const uint32_t last = (cur.x & kPairLastBit) ? kFlagLast : 0u;
                    if (ia >= n_a || ib < 0 || ib >= n_b) {
                        if (status_word) *status_word = BSP_ERR_DEVICE_RANGE;
                        ia = 0;
                        ib = 0;
                    }
                    const uint32_t ebar = empty_bar + 8 * lane;
                    const uint32_t fbar = full_bar + 8 * lane;
                    const uint32_t sa = data + lane * L::kStageBytes;
                    const uint32_t sb = sa + L::kBlockBytes;
                    PROF_T0(tw);
                    unsigned long long t0 = 0;
                    for (uint32_t spins = 1;; ++spins) {
                        if (mbar_try_wait(ebar, phase ^ 1u)) {
                            flags[lane] = last;
                            armed[lane] = (int)phase;
                            mbar_arrive_expect_tx(fbar, L::kStageBytes);
#pragma unroll
                            for (int h = 0; h < BS / 64; ++h) {
                                tma_load_2d(sa + h * (BS * 128), &map_a, h * 64, ia * BS, fbar);
                                tma_load_2d(sb + h * (BS * 128), &map_b, h * 64, ib * BS, fbar);
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
                    PROF_ADD(w_empty, tw);
                }
                alive = __all_sync(0xffffffffu, alive);
                phase ^= 1u;
                cur = nxt;
            }
            if (lane == 0) {
                PROF_STORE(0, clock64() - t_start);
                PROF_STORE(1, w_empty);
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                int stage = 0, acc = 0;
                uint32_t phase = 0, acc_phase = 0;
                bool first = true;
                PROF_DECL(w_full);
                PROF_DECL(w_tempty);
                PROF_T0(t_start);
                for (int pr = pr_begin; pr < pr_end; ++pr) {
                    if (first) {
                        PROF_T0(tw);
                        if (!mbar_wait(tempty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, status_word)) break;
                        PROF_ADD(w_tempty, tw);
                    }
                    PROF_T0(tw2);
                    if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, status_word)) break;
                    PROF_ADD(w_full, tw2);
                    tc_fence_after();
                    const uint32_t fl = flags[stage];
                    const uint32_t sa = data + stage * L::kStageBytes;
                    const uint32_t sb = sa + L::kBlockBytes;
                    const uint32_t d_tmem = tmem_base + acc * BS;
#pragma unroll
                    for (int k = 0; k < KSTEPS; ++k) {
                        tc_mma_f16(d_tmem, operand_desc<BS, A_MN>(sa, k), operand_desc<BS, B_MN>(sb, k),
                                   idesc, (first && k == 0) ? 0u : 1u);
                    }
                    tc_commit(empty_bar + 8 * stage);
                    first = false;
                    if (fl & kFlagLast) {
                        tc_commit(tfull_bar + 8 * acc);
                        first = true;
                        if (++acc == A) { acc = 0; acc_phase ^= 1u; }
                    }
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
                // make sure no MMA is still running before tensor memory is freed
                PROF_STORE(2, clock64() - t_start);
                PROF_STORE(3, w_full);
                PROF_STORE(4, w_tempty);
                tc_commit(drain_bar);
                mbar_wait(drain_bar, 0, abort_flag, status_word);
            }
        } else {
            // ---------------- epilogue ----------------
            const int q = warp & 3;  // tensor-memory subpartition of this warp
            constexpr int ROWS_PER_WARP = BS / 4;
            const bool row_valid = lane < ROWS_PER_WARP;
            const int row = q * ROWS_PER_WARP + lane;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool alive = true;
            PROF_DECL(w_tfull);
            PROF_T0(t_start);
            for (int w0 = blk_begin; w0 < blk_end && alive; w0 += 32) {
                const int bi = w0 + lane;
                const int my_n = bi < blk_end ? offsets[bi + 1] - offsets[bi] : 0;
                const int m = min(32, blk_end - w0);
                for (int j = 0; j < m && alive; ++j) {
                    const int n = __shfl_sync(0xffffffffu, my_n, j);
                    T* o = out + (int64_t)(w0 + j) * BS * BS;
                    if (n == 0) {
                        // this warp zeroes its quarter of the block
                        uint4* dst = reinterpret_cast<uint4*>(o + (int64_t)q * ROWS_PER_WARP * BS);
                        constexpr int VECS = ROWS_PER_WARP * BS * 2 / 16;
                        for (int i = lane; i < VECS; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
                        continue;
                    }
                    PROF_T0(tw);
                    if (!mbar_wait(tfull_bar + 8 * acc, acc_phase, abort_flag, status_word)) {
                        alive = false;
                    }
                    PROF_ADD(w_tfull, tw);
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + acc * BS + ((uint32_t)(q * 32) << 16);
#pragma unroll
                    for (int c0 = 0; c0 < BS; c0 += 32) {
                        uint32_t v[32];
                        tc_ld32(taddr + c0, v);
                        tc_wait_ld();
                        if (row_valid) {
                            // 32 columns = 64 bytes of the row: two 32-byte stores, each a whole sector
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
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);
                    if (++acc == A) { acc = 0; acc_phase ^= 1u; }
                }
            }
            if (warp == 2 && lane == 0) {
                PROF_STORE(5, clock64() - t_start);
                PROF_STORE(6, w_tfull);
                PROF_STORE(7, (long long)(pr_end - pr_begin) * 100000 + (blk_end - blk_begin));
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // bounded wait for copies that were issued but never consumed
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
                     ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
    }
}

// ---- host side -------------------------------------------------------------

template <typename T, int BS, int OP>
int launch_cfg(const CUtensorMap& ma, const CUtensorMap& mb, int64_t n_a, int64_t n_b, void* out,
               const int32_t* offsets, const int32_t* pairs, const int32_t* chunk_begin,
               int32_t n_chunks, int dtype, int32_t* status_word, cudaStream_t stream) {
    auto kern = matmul_umma_kernel<T, BS, OP>;
    constexpr int smem = SmemLayout<BS>::kTotal;
    BSP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<n_chunks, kThreads, smem, stream>>>(ma, mb, n_a, n_b, (T*)out, offsets, pairs, chunk_begin,
                                               make_idesc(dtype, BS, OP), status_word);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

template <typename T, int BS>
int launch_op(int op, const CUtensorMap& ma, const CUtensorMap& mb, int64_t n_a, int64_t n_b, void* out,
              const int32_t* offsets, const int32_t* pairs, const int32_t* chunk_begin, int32_t n_chunks,
              int dtype, int32_t* status_word, cudaStream_t stream) {
    switch (op) {
        case BSP_OP_NN: return launch_cfg<T, BS, BSP_OP_NN>(ma, mb, n_a, n_b, out, offsets, pairs, chunk_begin, n_chunks, dtype, status_word, stream);
        case BSP_OP_NT: return launch_cfg<T, BS, BSP_OP_NT>(ma, mb, n_a, n_b, out, offsets, pairs, chunk_begin, n_chunks, dtype, status_word, stream);
        case BSP_OP_TN: return launch_cfg<T, BS, BSP_OP_TN>(ma, mb, n_a, n_b, out, offsets, pairs, chunk_begin, n_chunks, dtype, status_word, stream);
        default: return BSP_ERR_INVALID_ARG;
    }
}

}  // namespace

#ifdef BSP_UMMA_PROFILE
extern "C" int bsp_debug_read_prof(long long* host_out, int n) {
    return (int)cudaMemcpyFromSymbol(host_out, g_prof, sizeof(long long) * n);
}
#endif

bool umma_applicable(int dtype, int bs) {
    return (dtype == BSP_F16 || dtype == BSP_BF16) && (bs == 64 || bs == 128);
}

int umma_num_chunks(int dtype, int bs) {
    if (!umma_applicable(dtype, bs)) return 0;
    return num_sms() * (bs == 64 ? Cfg<64>::kCtasPerSm : Cfg<128>::kCtasPerSm);
}

int launch_matmul_umma(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                       int64_t n_out, const int32_t* offsets, const int32_t* pairs,
                       const int32_t* chunk_begin, int32_t n_chunks, int bs, int dtype, int op,
                       int32_t* status_word, cudaStream_t stream) {
    if (!umma_applicable(dtype, bs)) return BSP_ERR_UNSUPPORTED;
    if (!chunk_begin || n_chunks < 1 || n_a < 1 || n_b < 1) return BSP_ERR_INVALID_ARG;
    // TMA coordinates are 32-bit row indices into the (n_blocks * bs)-row view.
    if (n_a * bs > 0x7fffffffLL || n_b * bs > 0x7fffffffLL || n_out > 0x7fffffffLL)
        return BSP_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15))
        return BSP_ERR_INVALID_ARG;
    CUtensorMap ma, mb;
    int st = make_block_map(&ma, a, n_a, bs, dtype);
    if (st != BSP_OK) return st;
    st = make_block_map(&mb, b, n_b, bs, dtype);
    if (st != BSP_OK) return st;
    if (dtype == BSP_F16) {
        if (bs == 64) return launch_op<__half, 64>(op, ma, mb, n_a, n_b, out, offsets, pairs, chunk_begin, n_chunks, dtype, status_word, stream);
        return launch_op<__half, 128>(op, ma, mb, n_a, n_b, out, offsets, pairs, chunk_begin, n_chunks, dtype, status_word, stream);
    }
    if (bs == 64) return launch_op<__nv_bfloat16, 64>(op, ma, mb, n_a, n_b, out, offsets, pairs, chunk_begin, n_chunks, dtype, status_word, stream);
    return launch_op<__nv_bfloat16, 128>(op, ma, mb, n_a, n_b, out, offsets, pairs, chunk_begin, n_chunks, dtype, status_word, stream);
}

}  // namespace bsp
