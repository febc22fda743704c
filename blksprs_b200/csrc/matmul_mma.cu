// Block-sparse matmul on a pair plan with warp-level mma.sync tensor-core
// instructions.  Serves the block sizes 16 and 32 (too small for a tcgen05
// tile) and fp32 data (TF32 mma, like the reference's tl.dot on fp32 inputs,
// blksprs/ops/matmul.py:242), and any other (dtype, bs) when asked for by
// BSP_KERNEL_MMA.
//
// Three kernels.
//
// matmul_mma_direct_kernel (block sizes 16 and 32, except fp32 blocks of 32): persistent CTAs of
// four warps; every warp works on its own and moves operand blocks from global memory straight into
// the registers that feed mma.sync, without shared memory or barriers (see the comment above it).
//
// matmul_mma_stream_kernel (fp32 blocks of 32): the same warp-autonomous walk over chunks of up to
// 32 consecutive output blocks, but with a ring of cp.async stages in shared memory per warp (one
// stage = the two operand blocks of a pair), several pairs ahead and across output-block
// boundaries, with the pair records fetched 32 at a time.
//
// matmul_mma_kernel (any block size; used for >= 64 when this family is asked for): one CTA
// computes one TILE x TILE tile of one output block, double-buffered cp.async per (pair, k-chunk).
//
// In the first two a block's result goes from the accumulator fragments straight to global memory
// and block boundaries come from the offsets array; no CTA-wide barrier exists in their loops.
//
// The two shared-memory kernels copy operand tiles in their global orientation; whether an operand
// is read transposed (BSP_OP_NT / BSP_OP_TN) is decided when the fragments are read from shared
// memory (ldmatrix[.trans] for 16-bit data, scalar loads for fp32).
#include "common.cuh"

namespace bsp {

template <typename T> struct Elem;
template <> struct Elem<__half> {
    static constexpr bool k16 = true;
    __device__ static inline void mma(float* c, const uint32_t* a, const uint32_t* b) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    __device__ static inline void store2(__half* p, float x, float y) {
        *reinterpret_cast<__half2*>(p) = __floats2half2_rn(x, y);
    }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr bool k16 = true;
    __device__ static inline void mma(float* c, const uint32_t* a, const uint32_t* b) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    __device__ static inline void store2(__nv_bfloat16* p, float x, float y) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
    }
};
template <> struct Elem<float> {
    static constexpr bool k16 = false;
    __device__ static inline void mma(float* c, const uint32_t* a, const uint32_t* b) {
        asm volatile(
            "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    __device__ static inline void store2(float* p, float x, float y) {
        *reinterpret_cast<float2*>(p) = make_float2(x, y);
    }
};

__device__ inline uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ inline void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ inline void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
// fp32 operands go to the TF32 tensor-core instruction as they are: the hardware reads the
// upper 19 bits and drops the low 13 mantissa bits.  This is what the reference's `tl.dot` on
// fp32 inputs does (blksprs/ops/matmul.py:242 with Triton's default input precision), and it makes
// fp32 results identical to the reference's on the same GPU; rounding to nearest instead would be
// closer to IEEE fp32 but about 1e-3 * max|ref| away from the reference.
__device__ inline uint32_t f32_to_tf32(float x) { return __float_as_uint(x); }
__device__ inline void ldmatrix_x4(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ inline void ldmatrix_x4_trans(uint32_t* r, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

// Row padding (in elements) of a shared-memory operand tile.  16-bit tiles are
// read with ldmatrix (8 rows of 16 B must fall into distinct bank groups: +16 B).
// fp32 tiles are read with scalar loads; a tile read along its rows by the
// fragment's 8-wide index wants a stride of 4 (mod 32) words, one read along
// its columns wants 8 (mod 32).
template <typename T, bool FRAG_ROWS_ARE_8WIDE>
struct Pad {
    static constexpr int value = sizeof(T) == 2 ? 8 : (FRAG_ROWS_ARE_8WIDE ? 4 : 8);
};

template <typename T, int TILE, int OP>
__global__ void __launch_bounds__(TILE == 16 ? 32 : 128)
matmul_mma_kernel(const T* __restrict__ a, int64_t n_a, const T* __restrict__ b, int64_t n_b,
                  T* __restrict__ out, const int32_t* __restrict__ offsets,
                  const int32_t* __restrict__ pairs, int bs, int32_t* __restrict__ status_word) {
    constexpr bool A_TRANS = (OP == BSP_OP_TN);  // shared A tile holds [k][m]
    constexpr bool B_NK = (OP == BSP_OP_NT);     // shared B tile holds [n][k]
    constexpr int NW = TILE == 16 ? 1 : 4;
    constexpr int NT = NW * 32;
    constexpr int WM = TILE == 16 ? 16 : TILE / 2;
    constexpr int WN = TILE == 16 ? 16 : TILE / 2;
    constexpr int MI = WM / 16, NI = WN / 8;
    constexpr int APAD = Pad<T, !A_TRANS>::value;
    constexpr int BPAD = Pad<T, B_NK>::value;
    constexpr int ALD = TILE + APAD, BLD = TILE + BPAD;
    constexpr int KSTEP = Elem<T>::k16 ? 16 : 8;
    constexpr int CHUNK = 16 / sizeof(T);  // elements per 16-byte copy

    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* As = reinterpret_cast<T*>(smem_raw);  // [2][TILE][ALD]
    T* Bs = As + 2 * TILE * ALD;             // [2][TILE][BLD]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = NW == 1 ? 0 : warp >> 1, warp_n = NW == 1 ? 0 : warp & 1;
    const int g = lane >> 2, t4 = lane & 3;

    const int64_t p = blockIdx.x;
    const int tiles = bs / TILE;
    const int tm = blockIdx.y / tiles, tn = blockIdx.y % tiles;
    const int beg = offsets[p], end = offsets[p + 1];
    const int nkc = bs / TILE;
    const int nsteps = (end - beg) * nkc;
    const int64_t blk_elems = (int64_t)bs * bs;

    float acc[MI][NI][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.f;

    // Copies the operand tiles of step s into buffer `buf`; returns false (and
    // copies nothing) when the pair's indices are out of range.
    auto issue = [&](int s, int buf) -> bool {
        const int pr = beg + s / nkc, kc = s % nkc;
        const int ia = pairs[2 * (int64_t)pr] & 0x3fffffff, ib = pairs[2 * (int64_t)pr + 1];
        const bool ok = ia >= 0 && ia < n_a && ib >= 0 && ib < n_b;
        if (ok) {
            const int ar0 = A_TRANS ? kc * TILE : tm * TILE, ac0 = A_TRANS ? tm * TILE : kc * TILE;
            const int br0 = B_NK ? tn * TILE : kc * TILE, bc0 = B_NK ? kc * TILE : tn * TILE;
            const T* ga = a + ia * blk_elems + (int64_t)ar0 * bs + ac0;
            const T* gb = b + ib * blk_elems + (int64_t)br0 * bs + bc0;
            T* sa = As + buf * TILE * ALD;
            T* sb = Bs + buf * TILE * BLD;
            constexpr int CPR = TILE / CHUNK;  // 16-byte copies per tile row
            for (int i = tid; i < TILE * CPR; i += NT) {
                const int r = i / CPR, c = (i % CPR) * CHUNK;
                cp_async16(sa + r * ALD + c, ga + (int64_t)r * bs + c);
                cp_async16(sb + r * BLD + c, gb + (int64_t)r * bs + c);
            }
        } else if (status_word && tid == 0) {
            *status_word = BSP_ERR_DEVICE_RANGE;
        }
        cp_async_commit();
        return ok;
    };

    bool ok_cur = false, ok_next = false;
    if (nsteps > 0) ok_cur = issue(0, 0);
    for (int s = 0; s < nsteps; ++s) {
        const int buf = s & 1;
        if (s + 1 < nsteps) {
            ok_next = issue(s + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (ok_cur) {
            const T* sa = As + buf * TILE * ALD;
            const T* sb = Bs + buf * TILE * BLD;
#pragma unroll
            for (int k0 = 0; k0 < TILE; k0 += KSTEP) {
                uint32_t af[MI][4];
                uint32_t bf[NI][2];
                if constexpr (Elem<T>::k16) {
                    const int q = lane >> 3, rr = lane & 7;
#pragma unroll
                    for (int i = 0; i < MI; ++i) {
                        const int m0 = warp_m * WM + i * 16;
                        if constexpr (!A_TRANS) {
                            ldmatrix_x4(af[i], sa + (m0 + rr + (q & 1) * 8) * ALD + k0 + (q >> 1) * 8);
                        } else {
                            ldmatrix_x4_trans(af[i], sa + (k0 + rr + (q >> 1) * 8) * ALD + m0 + (q & 1) * 8);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < NI; j += 2) {
                        const int n0 = warp_n * WN + j * 8;
                        uint32_t r4[4];
                        if constexpr (B_NK) {
                            ldmatrix_x4(r4, sb + (n0 + rr + (q >> 1) * 8) * BLD + k0 + (q & 1) * 8);
                        } else {
                            ldmatrix_x4_trans(r4, sb + (k0 + rr + (q & 1) * 8) * BLD + n0 + (q >> 1) * 8);
                        }
                        bf[j][0] = r4[0]; bf[j][1] = r4[1];
                        bf[j + 1][0] = r4[2]; bf[j + 1][1] = r4[3];
                    }
                } else {
                    auto A_at = [&](int m, int k) -> float {
                        return A_TRANS ? (float)sa[k * ALD + m] : (float)sa[m * ALD + k];
                    };
                    auto B_at = [&](int k, int n) -> float {
                        return B_NK ? (float)sb[n * BLD + k] : (float)sb[k * BLD + n];
                    };
#pragma unroll
                    for (int i = 0; i < MI; ++i) {
                        const int m0 = warp_m * WM + i * 16;
                        af[i][0] = f32_to_tf32(A_at(m0 + g, k0 + t4));
                        af[i][1] = f32_to_tf32(A_at(m0 + g + 8, k0 + t4));
                        af[i][2] = f32_to_tf32(A_at(m0 + g, k0 + t4 + 4));
                        af[i][3] = f32_to_tf32(A_at(m0 + g + 8, k0 + t4 + 4));
                    }
#pragma unroll
                    for (int j = 0; j < NI; ++j) {
                        const int n0 = warp_n * WN + j * 8;
                        bf[j][0] = f32_to_tf32(B_at(k0 + t4, n0 + g));
                        bf[j][1] = f32_to_tf32(B_at(k0 + t4 + 4, n0 + g));
                    }
                }
#pragma unroll
                for (int i = 0; i < MI; ++i)
#pragma unroll
                    for (int j = 0; j < NI; ++j) Elem<T>::mma(acc[i][j], af[i], bf[j]);
            }
        }
        __syncthreads();
        ok_cur = ok_next;
    }

    T* o = out + p * blk_elems;
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j) {
            const int row = tm * TILE + warp_m * WM + i * 16 + g;
            const int col = tn * TILE + warp_n * WN + j * 8 + 2 * t4;
            Elem<T>::store2(o + (int64_t)row * bs + col, acc[i][j][0], acc[i][j][1]);
            Elem<T>::store2(o + (int64_t)(row + 8) * bs + col, acc[i][j][2], acc[i][j][3]);
        }
}


// ---- warp-autonomous streaming kernel for block sizes 16 and 32 ----------------------------

template <typename T, int BS> struct StreamCfg {
    // Ring depth per warp, kept short to fit more warps per SM (fp32 blocks of 32, the one case this
    // kernel serves: two stages of 8.5 KiB per warp, 12 warps per SM).
    static constexpr int kStages = sizeof(T) == 2 ? (BS == 16 ? 4 : 3) : (BS == 16 ? 3 : 2);
    static constexpr int kWarps = 4;
};

template <typename T, int BS, int OP>
__global__ void __launch_bounds__(128)
matmul_mma_stream_kernel(const T* __restrict__ a, int64_t n_a, const T* __restrict__ b, int64_t n_b,
                         T* __restrict__ out, const int32_t* __restrict__ offsets,
                         const int32_t* __restrict__ pairs, int n_out, int chunk,
                         int32_t* __restrict__ status_word) {
    constexpr bool A_TRANS = (OP == BSP_OP_TN);  // shared A tile holds [k][m]
    constexpr bool B_NK = (OP == BSP_OP_NT);     // shared B tile holds [n][k]
    constexpr int S = StreamCfg<T, BS>::kStages;
    constexpr int MI = BS / 16, NI = BS / 8;
    constexpr int APAD = Pad<T, !A_TRANS>::value, BPAD = Pad<T, B_NK>::value;
    constexpr int ALD = BS + APAD, BLD = BS + BPAD;
    constexpr int KSTEP = Elem<T>::k16 ? 16 : 8;
    constexpr int CHUNK = 16 / sizeof(T);        // elements per 16-byte copy
    constexpr int CPR = BS / CHUNK;              // 16-byte copies per tile row
    constexpr int STAGE_ELEMS = BS * (ALD + BLD);
    constexpr int64_t BLK = (int64_t)BS * BS;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T* ring = reinterpret_cast<T*>(smem_raw) + (size_t)warp * S * STAGE_ELEMS;
    const int g = lane >> 2, t4 = lane & 3;
    const int total_warps = gridDim.x * StreamCfg<T, BS>::kWarps;
    const int n_chunks = (n_out + chunk - 1) / chunk;

    float acc[MI][NI][4];
    auto clear_acc = [&]() {
#pragma unroll
        for (int i = 0; i < MI; ++i)
#pragma unroll
            for (int j = 0; j < NI; ++j)
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.f;
    };
    auto write_block = [&](int64_t p) {
        T* o = out + p * BLK;
#pragma unroll
        for (int i = 0; i < MI; ++i)
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                const int row = i * 16 + g, col = j * 8 + 2 * t4;
                Elem<T>::store2(o + row * BS + col, acc[i][j][0], acc[i][j][1]);
                Elem<T>::store2(o + (row + 8) * BS + col, acc[i][j][2], acc[i][j][3]);
            }
    };

    for (int c = blockIdx.x * StreamCfg<T, BS>::kWarps + warp; c < n_chunks; c += total_warps) {
        const int p0 = c * chunk;
        const int nb = min(chunk, n_out - p0);
        // lane l holds the offset of block p0 + l (chunk <= 32); the range's end is read by all
        const int my_off = offsets[p0 + min(lane, nb)];
        const int q_begin = __shfl_sync(0xffffffffu, my_off, 0);
        const int q_end = offsets[p0 + nb];
        // without operand blocks there is nothing to multiply: every block of the chunk is written as zeros
        const int n_pairs = (n_a > 0 && n_b > 0) ? q_end - q_begin : 0;

        // pair records, 32 at a time: this window and the next one
        auto load_window = [&](int w) -> int2 {
            const int q = q_begin + w * 32 + lane;
            if (q < q_end) return *reinterpret_cast<const int2*>(pairs + 2 * (int64_t)q);
            return make_int2(-1, -1);
        };
        // `win` holds the window the copies are being issued from, `win_next` the one after it (in
        // flight for 32 issues before its first record is needed)
        int2 win = load_window(0), win_next = load_window(1);
        int win_no = 0;
        // the record of the next position to be issued is fetched (two shuffles) right after the previous
        // issue, so that its latency is hidden behind the multiplications in between
        int nia = 0, nib = 0;
        auto fetch_record = [&](int s) {
            if ((s >> 5) > win_no) {
                win = win_next;
                ++win_no;
                win_next = load_window(win_no + 1);
            }
            const int xa = __shfl_sync(0xffffffffu, win.x, s & 31);
            nib = __shfl_sync(0xffffffffu, win.y, s & 31);
            nia = xa & 0x3fffffff;  // bit 30 marks a block's last pair (not used here); a negative value stays out of range
        };
        // copies the two operand blocks of stream position s into its ring stage and commits the group;
        // beyond the end of the stream only an empty group is committed, which keeps the group count
        // per iteration constant.  Indices outside the operands are reported in the status word and
        // replaced by block 0 (which exists whenever a pair does), so that the access stays inside the
        // operands and the loop needs no special case.
        auto issue = [&](int s) {
            if (s < n_pairs) {
                int ia = nia, ib = nib;
                if ((unsigned)ia >= (unsigned long long)n_a || (unsigned)ib >= (unsigned long long)n_b) {
                    if (status_word && lane == 0) *status_word = BSP_ERR_DEVICE_RANGE;
                    ia = ib = 0;
                }
                const T* ga = a + ia * BLK;
                const T* gb = b + ib * BLK;
                T* sa = ring + (s % S) * STAGE_ELEMS;
                T* sb = sa + BS * ALD;
#pragma unroll
                for (int i = lane; i < BS * CPR; i += 32) {
                    const int r = i / CPR, cc = (i % CPR) * CHUNK;
                    cp_async16(sa + r * ALD + cc, ga + r * BS + cc);
                    cp_async16(sb + r * BLD + cc, gb + r * BS + cc);
                }
                if (s + 1 < n_pairs) fetch_record(s + 1);
            }
            cp_async_commit();
        };

        clear_acc();
        int blk = 0;  // current block, relative to p0
        // stream position at which block `bl` ends: the offsets of blocks p0 .. p0 + nb - 1 are in the
        // lanes, the last block ends with the range
        auto block_end = [&](int bl) {
            const int e = __shfl_sync(0xffffffffu, my_off, min(bl + 1, 31));
            return bl + 1 >= nb ? n_pairs : e - q_begin;
        };
        int blk_end = block_end(0);

        // fragments of one k-step of the pair in ring stage `st`
        auto load_frags = [&](int st, int k0, uint32_t (&af)[MI][4], uint32_t (&bf)[NI][2]) {
            const T* sa = ring + st * STAGE_ELEMS;
            const T* sb = sa + BS * ALD;
            if constexpr (Elem<T>::k16) {
                const int q = lane >> 3, rr = lane & 7;
#pragma unroll
                for (int i = 0; i < MI; ++i) {
                    const int m0 = i * 16;
                    if constexpr (!A_TRANS) {
                        ldmatrix_x4(af[i], sa + (m0 + rr + (q & 1) * 8) * ALD + k0 + (q >> 1) * 8);
                    } else {
                        ldmatrix_x4_trans(af[i], sa + (k0 + rr + (q >> 1) * 8) * ALD + m0 + (q & 1) * 8);
                    }
                }
#pragma unroll
                for (int j = 0; j < NI; j += 2) {
                    const int n0 = j * 8;
                    uint32_t r4[4];
                    if constexpr (B_NK) {
                        ldmatrix_x4(r4, sb + (n0 + rr + (q >> 1) * 8) * BLD + k0 + (q & 1) * 8);
                    } else {
                        ldmatrix_x4_trans(r4, sb + (k0 + rr + (q & 1) * 8) * BLD + n0 + (q >> 1) * 8);
                    }
                    bf[j][0] = r4[0]; bf[j][1] = r4[1];
                    bf[j + 1][0] = r4[2]; bf[j + 1][1] = r4[3];
                }
            } else {
                auto A_at = [&](int m, int k) -> float {
                    return A_TRANS ? (float)sa[k * ALD + m] : (float)sa[m * ALD + k];
                };
                auto B_at = [&](int k, int n) -> float {
                    return B_NK ? (float)sb[n * BLD + k] : (float)sb[k * BLD + n];
                };
#pragma unroll
                for (int i = 0; i < MI; ++i) {
                    const int m0 = i * 16;
                    af[i][0] = f32_to_tf32(A_at(m0 + g, k0 + t4));
                    af[i][1] = f32_to_tf32(A_at(m0 + g + 8, k0 + t4));
                    af[i][2] = f32_to_tf32(A_at(m0 + g, k0 + t4 + 4));
                    af[i][3] = f32_to_tf32(A_at(m0 + g + 8, k0 + t4 + 4));
                }
#pragma unroll
                for (int j = 0; j < NI; ++j) {
                    const int n0 = j * 8;
                    bf[j][0] = f32_to_tf32(B_at(k0 + t4, n0 + g));
                    bf[j][1] = f32_to_tf32(B_at(k0 + t4 + 4, n0 + g));
                }
            }
        };
        auto multiply = [&](const uint32_t (&af)[MI][4], const uint32_t (&bf)[NI][2]) {
#pragma unroll
            for (int i = 0; i < MI; ++i)
#pragma unroll
                for (int j = 0; j < NI; ++j) Elem<T>::mma(acc[i][j], af[i], bf[j]);
        };

        // S - 1 groups are committed ahead; every iteration commits one more, so that "at most S - 2
        // groups pending" always means: the group of position s has landed
        if (n_pairs > 0) fetch_record(0);
        for (int s = 0; s < S - 1; ++s) issue(s);
        for (int s = 0; s < n_pairs; ++s) {
            cp_async_wait<S - 2>();
            __syncwarp();
            // the first k-step's fragments are requested, then the copies of position s + S - 1 are issued
            // (into the stage that position s - 1 has finished with) while those loads are in flight
            uint32_t af[MI][4];
            uint32_t bf[NI][2];
            load_frags(s % S, 0, af, bf);
            issue(s + S - 1);
            // blocks that end before this pair (the previous pair's block, and empty ones) are written
            while (s == blk_end && blk < nb) {
                write_block(p0 + blk);
                clear_acc();
                ++blk;
                blk_end = block_end(blk);
            }
            multiply(af, bf);
#pragma unroll
            for (int k0 = KSTEP; k0 < BS; k0 += KSTEP) {
                load_frags(s % S, k0, af, bf);
                multiply(af, bf);
            }
            __syncwarp();  // all lanes are done with the stage before the next iteration refills it
        }
        cp_async_wait<0>();
        // the chunk's remaining blocks: the last one with pairs, and empty ones behind it
        while (blk < nb) {
            write_block(p0 + blk);
            clear_acc();
            ++blk;
        }
    }
}

template <typename T, int BS, int OP>
static int launch_stream(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out, int64_t n_out,
                         const int32_t* offsets, const int32_t* pairs, int32_t* status_word, cudaStream_t stream) {
    constexpr bool A_TRANS = (OP == BSP_OP_TN), B_NK = (OP == BSP_OP_NT);
    constexpr int ALD = BS + Pad<T, !A_TRANS>::value, BLD = BS + Pad<T, B_NK>::value;
    constexpr int W = StreamCfg<T, BS>::kWarps;
    constexpr size_t smem = (size_t)W * StreamCfg<T, BS>::kStages * BS * (ALD + BLD) * sizeof(T);
    auto kern = matmul_mma_stream_kernel<T, BS, OP>;
    // per device, looked up once: the shared-memory opt-in, the SM count and the resident CTAs per SM
    static int cached_sms[64] = {0}, cached_per_sm[64] = {0};
    int dev = 0;
    BSP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return BSP_ERR_UNSUPPORTED;
    if (cached_sms[dev] == 0) {
        int n_sm = 0, n_cta = 0;
        BSP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        BSP_CUDA_TRY(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
        BSP_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n_cta, kern, 32 * W, smem));
        cached_per_sm[dev] = n_cta < 1 ? 1 : n_cta;
        cached_sms[dev] = n_sm;
    }
    const int sms = cached_sms[dev], per_sm = cached_per_sm[dev];
    // chunks of consecutive output blocks per warp visit: as large as the block count allows while
    // every resident warp still gets several chunks (small problems: one block per warp)
    const int64_t warps = (int64_t)sms * per_sm * W;
    int64_t chunk = n_out / (warps * 4);
    chunk = chunk < 1 ? 1 : (chunk > 32 ? 32 : chunk);
    const int64_t n_chunks = (n_out + chunk - 1) / chunk;
    int64_t ctas = (n_chunks + W - 1) / W;
    if (ctas > (int64_t)sms * per_sm) ctas = (int64_t)sms * per_sm;
    kern<<<(unsigned)ctas, 32 * W, smem, stream>>>((const T*)a, n_a, (const T*)b, n_b, (T*)out, offsets, pairs,
                                                   (int)n_out, (int)chunk, status_word);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}


// ---- register-streaming kernel for block sizes 16 and 32 ------------------------------------
//
// Operand blocks go from global memory straight into the registers that feed mma.sync: no shared
// memory, no barrier.  What makes that possible is that a product does not care in which order
// its k terms are added, nor in which order its rows and columns are produced, as long as both
// operands agree on k and the result is stored where it belongs.
//
// Every lane (g = lane / 4, t4 = lane % 4) reads BS / 8 "row vectors" of each operand block: a row
// vector is the E = BS / 4 consecutive elements [E t4, E t4 + E) of one storage row, so four lanes
// read one whole row and a warp-wide load reads eight whole rows.  Vector r of a lane comes from
// row P(r) = E (g / 2) + 2 r + g % 2 ("permuted rows") or from row g + 8 r ("standard rows"); either
// way a lane's vectors are a fixed distance apart.  Then
//   * an operand stored with k along its rows (A of NN / NT, B of NT) already is an mma fragment
//     under the k assignment "k-step s, register half h of lane t4 = elements E t4 + 4 s + 2 h, + 1"
//     (16-bit data; E t4 + 2 s + h for tf32).  Its storage rows are m (n) indices: A uses standard
//     rows (a warp-wide load is one contiguous run), B permuted ones, which makes column tile j of
//     lane (g, t4) the output column E t4 + 2 j + {0, 1}: a lane's accumulators of one row are E
//     consecutive output elements and are written as one vector;
//   * a 16-bit operand stored with k along its columns (B of NN / TN, A of TN), read with permuted
//     rows, becomes the same fragment, with the same k assignment and the same column (row)
//     assignment, after one movmatrix (8 x 8 transposition across the warp) per register;
//   * fp32 operands with k along the columns cannot be transposed that way; they are read with
//     scalar loads in the standard fragment order (eight lanes = one 32-byte sector).
// A warp keeps D pairs in flight in registers (D * BS^2 / 8 bytes per lane); the residency of many
// warps per SM hides the rest of the latency.  On a product whose operands sit in L2 the kernel is
// bound by the L1 data path (operand vectors, movmatrix and the record shuffles all pass through it).

template <typename T, int BS> struct DirectCfg {
    static constexpr int kDepth = sizeof(T) == 2 ? (BS == 16 ? 4 : 2) : (BS == 16 ? 2 : 1);
    static constexpr int kWarps = 4;
    // resident CTAs per SM the register allocation is held to
    static constexpr int kMinCtas = sizeof(T) == 2 ? (BS == 16 ? 7 : 4) : (BS == 16 ? 6 : 3);
};

__device__ inline uint32_t movmatrix_trans(uint32_t x) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(x));
    return d;
}
template <int N>
__device__ inline void load_words(const char* p, uint32_t (&dst)[N]) {
    static_assert(N == 2 || N == 4 || N == 8, "vector of 8, 16 or 32 bytes");
    if constexpr (N == 2) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
        dst[0] = v.x; dst[1] = v.y;
    } else {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
            dst[4 * i] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
        }
    }
}
template <int N>
__device__ inline void store_words(char* p, const uint32_t (&src)[N]) {
    if constexpr (N == 2) {
        *reinterpret_cast<uint2*>(p) = make_uint2(src[0], src[1]);
    } else {
#pragma unroll
        for (int i = 0; i < N / 4; ++i)
            reinterpret_cast<uint4*>(p)[i] = make_uint4(src[4 * i], src[4 * i + 1], src[4 * i + 2], src[4 * i + 3]);
    }
}
__device__ inline uint32_t pack2(__half, float x, float y) {
    const __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ inline uint32_t pack2(__nv_bfloat16, float x, float y) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <typename T, int BS, int OP>
__global__ void __launch_bounds__(128, DirectCfg<T, BS>::kMinCtas)
matmul_mma_direct_kernel(const T* __restrict__ a, int64_t n_a, const T* __restrict__ b, int64_t n_b,
                         T* __restrict__ out, const int32_t* __restrict__ offsets,
                         const int32_t* __restrict__ pairs, int n_out, int chunk,
                         int32_t* __restrict__ status_word) {
    constexpr bool K16 = Elem<T>::k16;
    constexpr bool A_KROWS = (OP != BSP_OP_TN);  // A stored [m][k]
    constexpr bool B_KROWS = (OP == BSP_OP_NT);  // B stored [n][k]
    // 16-bit operands with k along the columns are transposed in registers ...
    constexpr bool A_MOVM = K16 && !A_KROWS, B_MOVM = K16 && !B_KROWS;
    // ... fp32 ones are read with scalar loads in the standard fragment order
    constexpr bool A_SCALAR = !K16 && !A_KROWS, B_SCALAR = !K16 && !B_KROWS;
    constexpr int D = DirectCfg<T, BS>::kDepth;
    constexpr int E = BS / 4;                          // elements of a row vector
    constexpr int R = BS / 8;                          // row vectors per lane and operand
    constexpr int X = E * (int)sizeof(T) / 4;          // 32-bit registers per row vector
    constexpr int MT = BS / 16, NT = BS / 8, KS = BS / (K16 ? 16 : 8);
    constexpr int ROW_BYTES = BS * (int)sizeof(T);
    constexpr int64_t BLK_BYTES = (int64_t)BS * ROW_BYTES;
    // Rows of the row vectors.  Where the row index is an m or n index that no transposition ties to
    // k, any assignment works, and "vector r = row g + 8 r" makes a warp-wide access one contiguous
    // run of eight rows.  A's rows are of that kind when A has k along its rows (they become the
    // result's rows); B's n rows (NT) are not, because the result's columns follow them.
    constexpr bool A_PROWS = A_MOVM;
    constexpr int A_VEC_STRIDE = (A_PROWS ? 2 : 8) * ROW_BYTES, B_VEC_STRIDE = 2 * ROW_BYTES;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int total_warps = gridDim.x * DirectCfg<T, BS>::kWarps;
    const int n_chunks = (n_out + chunk - 1) / chunk;
    // byte offsets, inside a block, of this lane's row vector 0 with permuted and with standard rows ...
    const int prow_off = (E * (g >> 1) + (g & 1)) * ROW_BYTES + E * t4 * (int)sizeof(T);
    const int srow_off = g * ROW_BYTES + E * t4 * (int)sizeof(T);
    // ... and of its first scalar element (fp32, k along the columns): row E t4, column g
    const int sca_off = E * t4 * ROW_BYTES + g * 4;
    const char* a_lane = reinterpret_cast<const char*>(a) + (A_SCALAR ? sca_off : A_PROWS ? prow_off : srow_off);
    const char* b_lane = reinterpret_cast<const char*>(b) + (B_SCALAR ? sca_off : prow_off);
    // the result: row vector r of this lane, in the rows A's assignment gives it
    char* out_lane = reinterpret_cast<char*>(out) + (A_PROWS ? prow_off : srow_off);
    // range limits as 32-bit values (a masked index is below 2^30, a negative one becomes huge)
    const uint32_t lim_a = (uint32_t)(n_a < 0x40000000LL ? n_a : 0x40000000LL);
    const uint32_t lim_b = (uint32_t)(n_b < 0x7fffffffLL ? n_b : 0x7fffffffLL);

    float acc[MT][NT][4];
    auto clear_acc = [&]() {
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.f;
    };
    auto write_block = [&](int64_t p) {
        char* o = out_lane + p * BLK_BYTES;
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r = 2 * i + u;
                if constexpr (!B_SCALAR) {
                    // E consecutive elements of one row
                    uint32_t w[X];
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        if constexpr (K16) {
                            w[j] = pack2(T(), acc[i][j][2 * u], acc[i][j][2 * u + 1]);
                        } else {
                            w[2 * j] = __float_as_uint(acc[i][j][2 * u]);
                            w[2 * j + 1] = __float_as_uint(acc[i][j][2 * u + 1]);
                        }
                    }
                    store_words<X>(o + r * A_VEC_STRIDE, w);
                } else {
                    // standard columns: two elements per column tile (out_lane points at column E t4 of the row)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
                        *reinterpret_cast<float2*>(o + r * A_VEC_STRIDE + (8 * j + 2 * t4 - E * t4) * 4) =
                            make_float2(acc[i][j][2 * u], acc[i][j][2 * u + 1]);
                }
            }
    };

    uint32_t ra[D][R][X], rb[D][R][X];
    auto load_operand = [&](const char* blk, const bool scalar, const int stride, uint32_t (&dst)[R][X]) {
        if (!scalar) {
#pragma unroll
            for (int r = 0; r < R; ++r) load_words<X>(blk + r * stride, dst[r]);
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int y = 0; y < X; ++y)
                    dst[r][y] = __ldg(reinterpret_cast<const uint32_t*>(blk + y * ROW_BYTES + 32 * r));
        }
    };
    // multiplies the pair held in a slot into the accumulators
    auto multiply = [&](uint32_t (&fa)[R][X], uint32_t (&fb)[R][X]) {
        if constexpr (A_MOVM) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int x = 0; x < X; ++x) fa[r][x] = movmatrix_trans(fa[r][x]);
        }
        if constexpr (B_MOVM) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int x = 0; x < X; ++x) fb[r][x] = movmatrix_trans(fb[r][x]);
        }
#pragma unroll
        for (int s = 0; s < KS; ++s) {
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                uint32_t af[4];
                if constexpr (A_MOVM) {
                    af[0] = fa[2 * s][2 * i]; af[1] = fa[2 * s][2 * i + 1];
                    af[2] = fa[2 * s + 1][2 * i]; af[3] = fa[2 * s + 1][2 * i + 1];
                } else {
                    af[0] = fa[2 * i][2 * s]; af[1] = fa[2 * i + 1][2 * s];
                    af[2] = fa[2 * i][2 * s + 1]; af[3] = fa[2 * i + 1][2 * s + 1];
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    uint32_t bf[2];
                    if constexpr (B_MOVM) {
                        bf[0] = fb[2 * s][j]; bf[1] = fb[2 * s + 1][j];
                    } else {
                        bf[0] = fb[j][2 * s]; bf[1] = fb[j][2 * s + 1];
                    }
                    Elem<T>::mma(acc[i][j], af, bf);
                }
            }
        }
    };
    // requests the operand blocks of a pair record into a slot.  Indices outside the operands are
    // reported in the status word and replaced by block 0 (which exists whenever a pair does).
    auto request = [&](const int2& win, int l, uint32_t (&fa)[R][X], uint32_t (&fb)[R][X]) {
        uint32_t ia = (uint32_t)__shfl_sync(0xffffffffu, win.x, l) & 0x3fffffffu;  // bit 30: a block's last pair
        uint32_t ib = (uint32_t)__shfl_sync(0xffffffffu, win.y, l);
        if (ia >= lim_a || ib >= lim_b) {
            if (status_word && lane == 0) *status_word = BSP_ERR_DEVICE_RANGE;
            ia = ib = 0;
        }
        load_operand(a_lane + (uint64_t)ia * (uint64_t)BLK_BYTES, A_SCALAR, A_VEC_STRIDE, fa);
        load_operand(b_lane + (uint64_t)ib * (uint64_t)BLK_BYTES, B_SCALAR, B_VEC_STRIDE, fb);
    };

    // A chunk: up to 32 consecutive output blocks, whose pairs are one contiguous range of the pair
    // list.  Lane l holds the offset of the chunk's block l; the range's end is held by all.
    struct Chunk { int p0, nb, my_off, q_end; };
    auto fetch_chunk = [&](int c) -> Chunk {
        Chunk k = {0, 0, 0, 0};
        if (c < n_chunks) {
            k.p0 = c * chunk;
            k.nb = min(chunk, n_out - k.p0);
            k.my_off = offsets[k.p0 + min(lane, k.nb)];
            k.q_end = offsets[k.p0 + k.nb];
        }
        return k;
    };
    // pair records of a chunk, 32 at a time: lane l of window w holds the record of stream position 32 w + l
    auto load_window = [&](int q_begin, int q_end, int w) -> int2 {
        const int q = q_begin + w * 32 + lane;
        if (q < q_end) return *reinterpret_cast<const int2*>(pairs + 2 * (int64_t)q);
        return make_int2(0, 0);
    };
    // without operand blocks there is nothing to multiply: every block is written as zeros
    const bool have_operands = n_a > 0 && n_b > 0;

    int c = blockIdx.x * DirectCfg<T, BS>::kWarps + warp;
    Chunk cur = fetch_chunk(c);
    int q_begin = __shfl_sync(0xffffffffu, cur.my_off, 0);
    int2 win = load_window(q_begin, cur.q_end, 0);
    int n_pairs = have_operands ? cur.q_end - q_begin : 0;
    // The pair stream of a chunk is walked by request position t: position t is requested into slot
    // t % D right after position t - D, which occupied that slot, has been multiplied; the walk runs
    // D positions past the stream's end.  The first D positions of a chunk are requested before the
    // chunk begins (here, and at the end of the chunk before it).
#pragma unroll
    for (int d = 0; d < D; ++d)
        if (d < n_pairs) request(win, d, ra[d], rb[d]);

    while (c < n_chunks) {
        // the next chunk's offsets travel while this chunk is worked on
        const Chunk nxt = fetch_chunk(c + total_warps);
        int2 nxt_win = make_int2(0, 0);
        int nxt_q_begin = 0;
        bool nxt_win_loaded = false;
        auto load_next_window = [&]() {
            nxt_q_begin = __shfl_sync(0xffffffffu, nxt.my_off, 0);
            nxt_win = load_window(nxt_q_begin, nxt.q_end, 0);
            nxt_win_loaded = true;
        };

        clear_acc();
        int blk = 0;  // current block, relative to p0
        // stream position at which block `bl` ends
        auto block_end = [&](int bl) {
            const int e = __shfl_sync(0xffffffffu, cur.my_off, min(bl + 1, 31));
            return bl + 1 >= cur.nb ? n_pairs : e - q_begin;
        };
        int blk_end = block_end(0);
        // one position (t >= D); CHECKED = false promises that t is inside the stream (then t - D is too)
        auto step = [&](const bool CHECKED, int t, uint32_t (&fa)[R][X], uint32_t (&fb)[R][X]) {
            const int s = t - D;
            if (!CHECKED || s < n_pairs) {
                // blocks that end before this pair (the previous pair's block, and empty ones) are written
                while (s == blk_end) {
                    write_block(cur.p0 + blk);
                    clear_acc();
                    ++blk;
                    blk_end = block_end(blk);
                }
                multiply(fa, fb);
            }
            if (!CHECKED || t < n_pairs) request(win, t & 31, fa, fb);
        };
        const int n_windows = (n_pairs + D + 31) >> 5;
        for (int w = 0; w < n_windows; ++w) {
            const int2 win_next = load_window(q_begin, cur.q_end, w + 1);
            // the next chunk's first records are asked for one window before they are needed
            if (w == n_windows - 1) load_next_window();
            const int base = w << 5;
            if (base + 32 <= n_pairs) {
                // window 0 starts behind the positions requested before the chunk began
#pragma unroll 1
                for (int tt = (w == 0 ? D : 0); tt < 32; tt += D) {
#pragma unroll
                    for (int d = 0; d < D; ++d) step(false, base + tt + d, ra[d], rb[d]);
                }
            } else {
#pragma unroll 1
                for (int tt = (w == 0 ? D : 0); tt < 32; tt += D) {
#pragma unroll
                    for (int d = 0; d < D; ++d) step(true, base + tt + d, ra[d], rb[d]);
                }
            }
            win = win_next;
        }
        if (!nxt_win_loaded) load_next_window();
        // all slots are free: the next chunk's first positions are requested before this chunk's last
        // blocks are written
        const int nxt_pairs = have_operands ? nxt.q_end - nxt_q_begin : 0;
#pragma unroll
        for (int d = 0; d < D; ++d)
            if (d < nxt_pairs) request(nxt_win, d, ra[d], rb[d]);
        // the chunk's remaining blocks: the last one with pairs, and empty ones behind it
        while (blk < cur.nb) {
            write_block(cur.p0 + blk);
            clear_acc();
            ++blk;
        }
        cur = nxt;
        win = nxt_win;
        q_begin = nxt_q_begin;
        n_pairs = nxt_pairs;
        c += total_warps;
    }
}

template <typename T, int BS, int OP>
static int launch_direct(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out, int64_t n_out,
                         const int32_t* offsets, const int32_t* pairs, int32_t* status_word, cudaStream_t stream) {
    constexpr int W = DirectCfg<T, BS>::kWarps;
    auto kern = matmul_mma_direct_kernel<T, BS, OP>;
    // per device, looked up once: the SM count and the resident CTAs per SM
    static int cached_sms[64] = {0}, cached_per_sm[64] = {0};
    int dev = 0;
    BSP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return BSP_ERR_UNSUPPORTED;
    if (cached_sms[dev] == 0) {
        int n_sm = 0, n_cta = 0;
        BSP_CUDA_TRY(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
        BSP_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n_cta, kern, 32 * W, 0));
        cached_per_sm[dev] = n_cta < 1 ? 1 : n_cta;
        cached_sms[dev] = n_sm;
    }
    const int sms = cached_sms[dev], per_sm = cached_per_sm[dev];
    // chunks of consecutive output blocks per warp visit: as large as the block count allows while
    // every resident warp still gets several chunks (small problems: one block per warp)
    const int64_t warps = (int64_t)sms * per_sm * W;
    int64_t chunk = n_out / (warps * 4);
    chunk = chunk < 1 ? 1 : (chunk > 32 ? 32 : chunk);
    const int64_t n_chunks = (n_out + chunk - 1) / chunk;
    int64_t ctas = (n_chunks + W - 1) / W;
    if (ctas > (int64_t)sms * per_sm) ctas = (int64_t)sms * per_sm;
    kern<<<(unsigned)ctas, 32 * W, 0, stream>>>((const T*)a, n_a, (const T*)b, n_b, (T*)out, offsets, pairs,
                                                (int)n_out, (int)chunk, status_word);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

// Block sizes 16 and 32: the register-streaming kernel, except for fp32 blocks of 32, whose 8 KiB per
// pair leave too few pairs in flight in registers (the shared-memory ring holds twice as many).
template <typename T, int BS, int OP>
static int launch_small(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out, int64_t n_out,
                        const int32_t* offsets, const int32_t* pairs, int32_t* status_word, cudaStream_t stream) {
    if constexpr (sizeof(T) == 4 && BS == 32)
        return launch_stream<T, BS, OP>(a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
    else
        return launch_direct<T, BS, OP>(a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
}

template <typename T, int BS>
static int launch_small_op(int op, const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                           int64_t n_out, const int32_t* offsets, const int32_t* pairs, int32_t* status_word,
                           cudaStream_t stream) {
    switch (op) {
        case BSP_OP_NN: return launch_small<T, BS, BSP_OP_NN>(a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
        case BSP_OP_NT: return launch_small<T, BS, BSP_OP_NT>(a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
        case BSP_OP_TN: return launch_small<T, BS, BSP_OP_TN>(a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
        default: return BSP_ERR_INVALID_ARG;
    }
}

template <typename T>
static int launch_small_bs(int bs, int op, const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                           int64_t n_out, const int32_t* offsets, const int32_t* pairs, int32_t* status_word,
                           cudaStream_t stream) {
    if (bs == 16) return launch_small_op<T, 16>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
    return launch_small_op<T, 32>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
}

template <typename T, int TILE, int OP>
static int launch_one(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                      int64_t n_out, const int32_t* offsets, const int32_t* pairs, int bs,
                      int32_t* status_word, cudaStream_t stream) {
    constexpr bool A_TRANS = (OP == BSP_OP_TN), B_NK = (OP == BSP_OP_NT);
    constexpr int ALD = TILE + Pad<T, !A_TRANS>::value, BLD = TILE + Pad<T, B_NK>::value;
    constexpr size_t smem = (size_t)2 * TILE * (ALD + BLD) * sizeof(T);
    auto kern = matmul_mma_kernel<T, TILE, OP>;
    if (smem > 48 * 1024)
        BSP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int tiles = bs / TILE;
    dim3 grid((unsigned)n_out, (unsigned)(tiles * tiles));
    kern<<<grid, TILE == 16 ? 32 : 128, smem, stream>>>((const T*)a, n_a, (const T*)b, n_b, (T*)out,
                                                         offsets, pairs, bs, status_word);
    BSP_LAUNCH_CHECK();
    return BSP_OK;
}

template <typename T, int TILE>
static int launch_op(int op, const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                     int64_t n_out, const int32_t* offsets, const int32_t* pairs, int bs,
                     int32_t* status_word, cudaStream_t stream) {
    switch (op) {
        case BSP_OP_NN: return launch_one<T, TILE, BSP_OP_NN>(a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
        case BSP_OP_NT: return launch_one<T, TILE, BSP_OP_NT>(a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
        case BSP_OP_TN: return launch_one<T, TILE, BSP_OP_TN>(a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
        default: return BSP_ERR_INVALID_ARG;
    }
}

template <typename T>
static int launch_tile(int op, const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                       int64_t n_out, const int32_t* offsets, const int32_t* pairs, int bs,
                       int32_t* status_word, cudaStream_t stream) {
    // fp32 tiles are capped at 32 to keep the double-buffered tiles small.
    const int cap = sizeof(T) == 4 ? 32 : 64;
    const int tile = bs < cap ? bs : cap;
    if (tile == 16) return launch_op<T, 16>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
    if (tile == 32) return launch_op<T, 32>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
    if constexpr (sizeof(T) == 2) {
        if (tile == 64) return launch_op<T, 64>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
    }
    return BSP_ERR_UNSUPPORTED;
}

int launch_matmul_mma(const void* a, int64_t n_a, const void* b, int64_t n_b, void* out,
                      int64_t n_out, const int32_t* offsets, const int32_t* pairs, int bs,
                      int dtype, int op, int32_t* status_word, cudaStream_t stream) {
    if (n_out > 0x7fffffffLL) return BSP_ERR_UNSUPPORTED;
    if (bs == 16 || bs == 32) {
        switch (dtype) {
            case BSP_F16: return launch_small_bs<__half>(bs, op, a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
            case BSP_BF16: return launch_small_bs<__nv_bfloat16>(bs, op, a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
            case BSP_F32: return launch_small_bs<float>(bs, op, a, n_a, b, n_b, out, n_out, offsets, pairs, status_word, stream);
            default: return BSP_ERR_UNSUPPORTED;
        }
    }
    const int tiles_cap = bs / (dtype == BSP_F32 ? 32 : 64);
    if (tiles_cap > 0 && (int64_t)tiles_cap * tiles_cap > 65535) return BSP_ERR_UNSUPPORTED;
    switch (dtype) {
        case BSP_F16: return launch_tile<__half>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
        case BSP_BF16: return launch_tile<__nv_bfloat16>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
        case BSP_F32: return launch_tile<float>(op, a, n_a, b, n_b, out, n_out, offsets, pairs, bs, status_word, stream);
        default: return BSP_ERR_UNSUPPORTED;
    }
}

}  // namespace bsp
