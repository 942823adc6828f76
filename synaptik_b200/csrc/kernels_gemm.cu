// GEMM kernels.
//
//  * gemm_exact_kernel: CUDA-core product whose every output cell is the reference's ascending-k
//    chain of separately rounded multiply and add (CpuMatmulReferenceKernel.java:71-93), so small
//    products are bit-identical to the reference CPU backend.  Strided operands and result.
//  * split kernels + gemm_tf32x3_kernel: the tensor-core path for large products.  FP32 operands
//    are split once into hi = tf32(x) and lo = tf32(x - hi) planes; the GEMM kernel is a persistent,
//    warp-specialised tcgen05 pipeline (TMA loads of 128-byte-swizzled K-major tiles -> UMMA
//    kind::tf32 with FP32 accumulators in tensor memory -> epilogue straight from tensor memory)
//    that issues lo*hi, hi*lo and hi*hi into one accumulator (3xTF32).  The dropped lo*lo term is
//    below 2^-22 of each product.
#include "kernels.hpp"
#include "activation.cuh"
#include "lowp.cuh"
#include "split.cuh"

#include <cuda.h>

#include <cstdio>
#include <cstdlib>

namespace syn {
namespace kern {

namespace {

// ------------------------------------------------------------------------------------------------
// Exact CUDA-core GEMM: 64x64 result tile, 16-deep k slices, 256 threads, 4x4 cells per thread.
// ------------------------------------------------------------------------------------------------
constexpr int XT = 64, XK = 16;

__global__ void __launch_bounds__(256) gemm_exact_kernel(int64_t m, int64_t n, int64_t k,
        const float *__restrict__ a, int64_t a_ms, int64_t a_ks, const float *__restrict__ b, int64_t b_ks, int64_t b_ns,
        float *c, int64_t c_ms, int64_t c_ns, GemmEpilogue ep) {
    __shared__ float as[XK][XT + 4];
    __shared__ float bs[XK][XT + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * XT, n0 = (int64_t)blockIdx.x * XT;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    const bool a_kfast = a_ks == 1, b_nfast = b_ns == 1;
    for (int64_t k0 = 0; k0 < k; k0 += XK) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            int e = tid + q * 256;
            int row = a_kfast ? e / XK : e % XT, kk = a_kfast ? e % XK : e / XT;
            int64_t gm = m0 + row, gk = k0 + kk;
            as[kk][row] = (gm < m && gk < k) ? a[gm * a_ms + gk * a_ks] : 0.0f;
            int col = b_nfast ? e % XT : e / XK, kb = b_nfast ? e / XT : e % XK;
            int64_t gn = n0 + col, gkb = k0 + kb;
            bs[kb][col] = (gn < n && gkb < k) ? b[gkb * b_ks + gn * b_ns] : 0.0f;
        }
        __syncthreads();
        const int depth = (int)((k - k0) < XK ? (k - k0) : XK);
        if (k == 1) {
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __fmul_rn(as[0][ty * 4 + i], bs[0][tx * 4 + j]);
        } else {
            for (int kk = 0; kk < depth; kk++) {
                float av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) av[i] = as[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; j++) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int64_t gm = m0 + ty * 4 + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int64_t gn = n0 + tx * 4 + j;
            if (gn >= n) continue;
            float z = acc[i][j];
            if (ep.bias) z = __fadd_rn(z, ep.bias[gn]);
            if (ep.gate) z = ep.gate[gm * n + gn] > 0.0f ? z : 0.0f;
            if (ep.second) { c[gm * c_ms + gn * c_ns] = z; ep.second[gm * n + gn] = activation_value(ep.act, z); }
            else c[gm * c_ms + gn * c_ns] = activation_value(ep.act, z);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// hi / lo split into zero-padded K-major planes.
// ------------------------------------------------------------------------------------------------
__global__ void split_rows_kernel(const float *__restrict__ src, int64_t rows, int64_t cols, int64_t rs,
                                  float *hi, float *lo, int64_t cp, int vec_ok) {
    const int64_t quads = cp >> 2, total = rows * quads;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / quads, c = (i - r * quads) << 2;
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float *p = src + r * rs + c;
        if (vec_ok && c + 3 < cols) { float4 v = *reinterpret_cast<const float4 *>(p); x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w; }
        else {
#pragma unroll
            for (int q = 0; q < 4; q++) if (c + q < cols) x[q] = p[q];
        }
        float h[4], l[4];
#pragma unroll
        for (int q = 0; q < 4; q++) split_value(x[q], h[q], l[q]);
        *reinterpret_cast<float4 *>(hi + r * cp + c) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4 *>(lo + r * cp + c) = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// ------------------------------------------------------------------------------------------------
// tcgen05 3xTF32 GEMM.
// ------------------------------------------------------------------------------------------------
constexpr int BM = 128;             // rows of P per tile = UMMA M = tensor-memory lanes
constexpr int BK = 32;              // floats per k-block: one 128-byte swizzle row
constexpr int KPAD = 32;            // planes are padded to a multiple of 32 columns
constexpr int UMMA_K = 8;           // kind::tf32 contracts 8 elements (32 bytes) per instruction
constexpr int GEMM_THREADS = 256;   // warp 0 TMA producer, warp 1 MMA issuer + tensor-memory owner, warps 4-7 epilogue
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // every device-side wait gives up after two seconds

template <int BN> struct TileConfig {
    static constexpr int kStages = BN == 256 ? 2 : (BN == 128 ? 3 : 4);
    static constexpr int kABytes = BM * BK * 4;            // one plane of P
    static constexpr int kBBytes = BN * BK * 4;            // one plane of Q
    static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;     // two accumulators, power of two
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t global_timer() { uint64_t t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: returns false (after raising the block's abort flag) when the phase has not
// completed within limit_ns or another role has already given up.
__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer();
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 63u) {
            if (*abort_flag) return false;
            if (global_timer() - start > limit_ns) { *abort_flag = 1; return false; }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    return mbar_wait_limited(bar, parity, abort_flag, WAIT_LIMIT_NS);
}

// The give-up path of the wait above, run on purpose: one warp waits for a phase of a barrier that
// nothing ever completes, the wait expires after limit_ns, and the kernel reports it the way the GEMM
// kernels do (abort flag -> ERR_WAIT_TIMEOUT in the context's error word) and returns normally.
__global__ void __launch_bounds__(32) wait_probe_kernel(uint64_t limit_ns, int *error_word) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait_limited(smem_u32(&bar), 0u, &abort_flag, limit_ns);
    __syncwarp();
    if (threadIdx.x == 0 && (!ok || abort_flag)) atomicOr(error_word, ERR_WAIT_TIMEOUT);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
// One operand tile of k-block kb starting at operand row r0 (a multiple of 32).  K-major planes are
// [rows, k]: a 2-D box at (k, row).  MN-major planes are [k, rows] seen through a 3-D map
// (32 rows, k, rows / 32): a box at (0, k, row / 32), whose first coordinate is always 0.
__device__ __forceinline__ void load_operand(uint32_t dst, const CUtensorMap *map, uint32_t bar, int kb, int r0, int mn_major) {
    if (mn_major) tma_load_3d(dst, map, bar, 0, kb * BK, r0 >> 5);
    else tma_load_2d(dst, map, bar, kb * BK, r0);
}

// Shared-memory matrix descriptors (descriptor version 1), two operand layouts.
// K-major: the tile is [rows][32 floats of k], 128-byte swizzle (layout type 2); each 128-byte row
//   holds one row's k-block, groups of 8 rows are 1024 bytes apart (stride offset); the leading offset
//   is unused and carries 1.  One MMA (8 contraction steps) advances the start address by 32 bytes
//   inside the swizzle row.
// MN-major: the tile is [rows / 32][32 k][32 floats of rows]; each 128-byte row holds 32 consecutive
//   rows of the operand at one k.  For 32-bit elements the tensor core reads this form only in the
//   128-byte swizzle with 32-byte atoms (layout type 1; the plain 128-byte swizzle returns zeros,
//   measured): the pattern repeats every 4 k, groups of 4 k are 512 bytes apart (stride offset) and the
//   next 32 operand rows start 4096 bytes later (leading offset).  One MMA covers 8 k = two groups and
//   advances the start address by 1024 bytes.  TMA writes the matching pattern with
//   CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.
struct OperandForm { uint64_t fixed; uint32_t k8_step; };
__device__ __forceinline__ OperandForm operand_form(int mn_major) {
    OperandForm f;
    if (mn_major) {
        f.fixed = ((uint64_t)((BK * 128u) >> 4) << 16) | ((uint64_t)(512u >> 4) << 32) | (1ull << 46) | (1ull << 61);
        f.k8_step = 1024u;
    } else {
        f.fixed = (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
        f.k8_step = (uint32_t)(UMMA_K * 4);
    }
    return f;
}
__device__ __forceinline__ uint64_t umma_desc(const OperandForm &f, uint32_t smem_addr) {
    return f.fixed | (uint64_t)((smem_addr & 0x3ffffu) >> 4);
}
// Instruction descriptor: FP32 accumulate, TF32 x TF32, M rows, N = BN columns, operand majors
// (bit 15: P is MN-major, bit 16: Q is MN-major).
__device__ __forceinline__ uint32_t umma_idesc(int rows, int bn, int p_mn, int q_mn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p_mn != 0) << 15) | ((uint32_t)(q_mn != 0) << 16)
           | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(rows >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_load32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

struct TcParams {
    float *d; int64_t ldd;
    int m, n, k_blocks;
    int tiles_m, tiles_n;
    const float *bias; const float *gate; float *second; int act;    // act: 0 none, else the activation's wire code
    float *nhi, *nlo; int64_t nld;          // optional [m, nld] hi/lo planes of the result
    int p_mn, q_mn;                          // operand planes are MN-major ([k, rows]) instead of K-major ([rows, k])
    int chunk_kb;                            // promoted kernel: k-blocks per tensor-memory partial sum
    int *error_word;
};
// Kept apart from TcParams on purpose: with 128 register sums per epilogue thread the 256-wide kernels
// sit at the edge of their register budget, and growing TcParams pushed ptxas into an allocation that
// ran the epilogue-bound K = 784 layer 40 % slower (measured).  After touching either struct compare
// -Xptxas -v: 204 bytes of spill stores / 224 of spill loads for the <256> two-SM kernel is the good state.
struct SliceParams {                         // two-SM kernel: split of the contraction into slices, tile order
    int slices, kb_per_slice;
    float *ws; int64_t ld;                   // workspace [slices][m][ld] of the slices' partial products
    int group_n;                             // tile columns per group (see tile_origin)
    int *unit_counter;                       // dynamic assignment: the next unit number, zero before the launch
};

// Tile order of the two-SM kernel.  The 74 pairs work on 74 consecutive tiles at a time.  In plain
// row-major order those cover every tile column and few row bands, so all of Q (134 MB of planes for a
// 4096 x 4096 weight) cycles through L2 once per few row bands and is read from DRAM again and again
// (measured: 16.7 GB per 65536 x 4096 x 4096 product whose operands are 2.3 GB).  Grouped order: the
// tile columns are cut into groups of group_n, and each group is swept down all row bands before the
// next group starts, so the tiles in flight share fewer distinct Q columns and more P row bands.
__device__ __forceinline__ void tile_origin(int tile, int tiles_m, int tiles_n, int group_n, int &mi, int &ni) {
    const int per_group = tiles_m * group_n;
    const int g = tile / per_group, within = tile - g * per_group;
    const int first = g * group_n;
    const int width = tiles_n - first < group_n ? tiles_n - first : group_n;     // the last group may be narrower
    mi = within / width;
    ni = first + (within - mi * width);
}


// The activations other than ReLU evaluate an elementary function in binary64 (activation.cuh).  Kept out
// of line and out of the kernels that never need them: inlined into the 32 call sites of an epilogue
// thread that holds 128 register sums they would take the registers the sums live in.
__device__ __noinline__ float4 activate4(int act, float4 z) {
    return make_float4(activation_value(act, z.x), activation_value(act, z.y), activation_value(act, z.z), activation_value(act, z.w));
}

// Finishes four adjacent result cells of one row: bias, ReLU-backward gate, activation, the stores
// of the result (and of the second output), and the hi/lo operand planes when later GEMMs read this
// result.  GENERAL: the activation may be any of the epilogue vocabulary; otherwise it is ReLU or none.
template <bool GENERAL>
__device__ __forceinline__ void epilogue_emit4(const TcParams &prm, int row, int col,
                                               float z0, float z1, float z2, float z3, bool vec_ok) {
    float *drow = prm.d + (int64_t)row * prm.ldd;
    const int64_t dense = (int64_t)row * prm.n;
    float z[4] = {z0, z1, z2, z3};
    float y[4];                             // the value later GEMMs read: activation or (gated) result
    if (col + 3 < prm.n && vec_ok && (prm.n & 3) == 0) {
        if (prm.bias) { float4 bv = *reinterpret_cast<const float4 *>(prm.bias + col);
            z[0] = __fadd_rn(z[0], bv.x); z[1] = __fadd_rn(z[1], bv.y); z[2] = __fadd_rn(z[2], bv.z); z[3] = __fadd_rn(z[3], bv.w); }
        if (prm.gate) { float4 gv = *reinterpret_cast<const float4 *>(prm.gate + dense + col);
            z[0] = gv.x > 0.0f ? z[0] : 0.0f; z[1] = gv.y > 0.0f ? z[1] : 0.0f; z[2] = gv.z > 0.0f ? z[2] : 0.0f; z[3] = gv.w > 0.0f ? z[3] : 0.0f; }
        if (GENERAL) {
            const float4 a = activate4(prm.act, make_float4(z[0], z[1], z[2], z[3]));
            y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) y[e] = prm.act ? relu_value(z[e]) : z[e];
        }
        if (prm.second) {
            *reinterpret_cast<float4 *>(drow + col) = make_float4(z[0], z[1], z[2], z[3]);
            *reinterpret_cast<float4 *>(prm.second + dense + col) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
            *reinterpret_cast<float4 *>(drow + col) = make_float4(y[0], y[1], y[2], y[3]);
        }
    } else {
        if (prm.bias) {
#pragma unroll
            for (int e = 0; e < 4; e++) if (col + e < prm.n) z[e] = __fadd_rn(z[e], prm.bias[col + e]);
        }
        if (prm.gate) {
#pragma unroll
            for (int e = 0; e < 4; e++) if (col + e < prm.n) z[e] = prm.gate[dense + col + e] > 0.0f ? z[e] : 0.0f;
        }
        if (GENERAL) {
            const float4 a = activate4(prm.act, make_float4(z[0], z[1], z[2], z[3]));
            y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) y[e] = prm.act ? relu_value(z[e]) : z[e];
        }
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int cc = col + e;
            if (cc < prm.n) {
                if (prm.second) { drow[cc] = z[e]; prm.second[dense + cc] = y[e]; }
                else drow[cc] = y[e];
            } else y[e] = 0.0f;
        }
    }
    if (prm.nhi) {
        // operand planes for the GEMMs that read this result, written here instead of by a separate
        // split pass; columns past n and rows past m are zero padding
        float h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; e++) split_value(y[e], h[e], l[e]);
        *reinterpret_cast<float4 *>(prm.nhi + (int64_t)row * prm.nld + col) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4 *>(prm.nlo + (int64_t)row * prm.nld + col) = make_float4(l[0], l[1], l[2], l[3]);
    }
}

template <int BN, bool GENERAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tf32x3_kernel(
        const __grid_constant__ CUtensorMap map_p_hi, const __grid_constant__ CUtensorMap map_p_lo,
        const __grid_constant__ CUtensorMap map_q_hi, const __grid_constant__ CUtensorMap map_q_lo, TcParams prm) {
    using Cfg = TileConfig<BN>;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle pattern
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S * Cfg::kStageBytes);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) accumulator full, [2S+2..2S+4) accumulator empty
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {        // one warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = prm.tiles_m * prm.tiles_n;
    const int kb_count = prm.k_blocks;
    const uint32_t smem_base = smem_u32(smem);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            uint32_t armed_phase[S]; bool armed[S];
            for (int s = 0; s < S; s++) { armed[s] = false; armed_phase[s] = 0; }
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / prm.tiles_n) * BM, n0 = (tile % prm.tiles_n) * BN;
                for (int kb = 0; kb < kb_count; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                    mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    armed[stage] = true; armed_phase[stage] = phase;
                    load_operand(sa, &map_p_hi, full_bar(stage), kb, m0, prm.p_mn);
                    load_operand(sa + Cfg::kABytes, &map_p_lo, full_bar(stage), kb, m0, prm.p_mn);
                    load_operand(sa + 2 * Cfg::kABytes, &map_q_hi, full_bar(stage), kb, n0, prm.q_mn);
                    load_operand(sa + 2 * Cfg::kABytes + Cfg::kBBytes, &map_q_lo, full_bar(stage), kb, n0, prm.q_mn);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok || *abort_flag) {
                // leave no bulk copy in flight towards this block's shared memory
                for (int s = 0; s < S; s++) if (armed[s]) mbar_wait(full_bar(s), armed_phase[s], abort_flag);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BM, BN, prm.p_mn, prm.q_mn);
            const OperandForm pf = operand_form(prm.p_mn), qf = operand_form(prm.q_mn);
            int stage = 0; uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, local++) {
                const int acc = local & 1;
                if (!mbar_wait(acc_empty_bar(acc), (((uint32_t)local >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < kb_count; kb++) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                    const uint32_t p_hi = sa, p_lo = sa + Cfg::kABytes, q_hi = sa + 2 * Cfg::kABytes, q_lo = q_hi + Cfg::kBBytes;
#pragma unroll
                    for (int k4 = 0; k4 < BK / UMMA_K; k4++) {
                        const uint32_t po = k4 * pf.k8_step, qo = k4 * qf.k8_step;
                        // small terms first, then the leading product
                        umma_tf32(tmem_d, umma_desc(pf, p_lo + po), umma_desc(qf, q_hi + qo), idesc, (kb | k4) != 0);
                        umma_tf32(tmem_d, umma_desc(pf, p_hi + po), umma_desc(qf, q_lo + qo), idesc, 1u);
                        umma_tf32(tmem_d, umma_desc(pf, p_hi + po), umma_desc(qf, q_hi + qo), idesc, 1u);
                    }
                    umma_commit(empty_bar(stage));          // releases the stage once these MMAs have read it
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(acc_full_bar(acc));     // accumulator complete
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue: tensor memory -> registers -> global ----------------
        const int quarter = warp & 3;                       // a warp may only touch lanes 32*(warp%4)..+31
        int local = 0;
        bool ok = true;
        const bool vec_ok = (prm.ldd & 3) == 0 && ((uintptr_t)prm.d & 15) == 0
                            && (!prm.second || ((uintptr_t)prm.second & 15) == 0) && (!prm.gate || ((uintptr_t)prm.gate & 15) == 0);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, local++) {
            const int acc = local & 1;
            const int m0 = (tile / prm.tiles_n) * BM, n0 = (tile % prm.tiles_n) * BN;
            ok = mbar_wait(acc_full_bar(acc), ((uint32_t)local >> 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);     // the warp-wide tensor-memory loads below need one verdict
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; chunk++) {
                float v[32];
                tmem_load32(taddr + (uint32_t)(chunk * 32), v);
                const int col0 = n0 + chunk * 32;
                const bool row_ok = row < prm.m;
                if (row_ok && col0 < prm.n) {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        epilogue_emit4<GENERAL>(prm, row, col0 + q * 4, v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3], vec_ok);
                }
            }
            tc_fence_before();
            mbar_arrive(acc_empty_bar(acc));
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(prm.error_word, ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// The same pipeline with FP32 promotion.  Measured on B200: every tcgen05.mma adds its products into
// the FP32 accumulator with truncation (toward zero), so a sum kept in tensor memory over the whole
// contraction drifts by about 0.2 * K units of 2^-24 of the running sum.  Here tensor memory only
// ever holds the partial sum of chunk_kb k-blocks (32 contraction steps each); eight epilogue warps
// add each finished partial into round-to-nearest FP32 register sums (128 per thread at BN = 256)
// while the tensor core already works on the next partial in the other tensor-memory buffer.
// The truncation is then relative to a short partial sum and the drift no longer grows with K.
// ------------------------------------------------------------------------------------------------
constexpr int PROMOTED_THREADS = 384;   // warp 0 producer, warp 1 MMA issuer, warps 4-11 epilogue

__device__ __forceinline__ void tmem_load16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}


template <int BN, bool GENERAL>
__global__ void __launch_bounds__(PROMOTED_THREADS, 1) gemm_tf32x3_promoted_kernel(
        const __grid_constant__ CUtensorMap map_p_hi, const __grid_constant__ CUtensorMap map_p_lo,
        const __grid_constant__ CUtensorMap map_q_hi, const __grid_constant__ CUtensorMap map_q_lo, TcParams prm) {
    using Cfg = TileConfig<BN>;
    constexpr int S = Cfg::kStages;
    constexpr int CPT = BN / 2;             // result columns per epilogue thread
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S * Cfg::kStageBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 256); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = prm.tiles_m * prm.tiles_n;
    const int kb_count = prm.k_blocks;
    const int CHUNK_KB = prm.chunk_kb;
    const uint32_t smem_base = smem_u32(smem);

    // the two epilogue warpgroups hold the register sums: hand them the registers the producer /
    // issuer warpgroup does not need
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            uint32_t armed_phase[S]; bool armed[S];
            for (int s = 0; s < S; s++) { armed[s] = false; armed_phase[s] = 0; }
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / prm.tiles_n) * BM, n0 = (tile % prm.tiles_n) * BN;
                for (int kb = 0; kb < kb_count; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                    mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    armed[stage] = true; armed_phase[stage] = phase;
                    load_operand(sa, &map_p_hi, full_bar(stage), kb, m0, prm.p_mn);
                    load_operand(sa + Cfg::kABytes, &map_p_lo, full_bar(stage), kb, m0, prm.p_mn);
                    load_operand(sa + 2 * Cfg::kABytes, &map_q_hi, full_bar(stage), kb, n0, prm.q_mn);
                    load_operand(sa + 2 * Cfg::kABytes + Cfg::kBBytes, &map_q_lo, full_bar(stage), kb, n0, prm.q_mn);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok || *abort_flag) {
                for (int s = 0; s < S; s++) if (armed[s]) mbar_wait(full_bar(s), armed_phase[s], abort_flag);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BM, BN, prm.p_mn, prm.q_mn);
            const OperandForm pf = operand_form(prm.p_mn), qf = operand_form(prm.q_mn);
            int stage = 0; uint32_t phase = 0;
            uint32_t partial = 0;               // running count of partial sums: selects the tensor-memory buffer
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                for (int kb0 = 0; kb0 < kb_count && ok; kb0 += CHUNK_KB, partial++) {
                    const int buf = partial & 1;
                    if (!mbar_wait(acc_empty_bar(buf), ((partial >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                    const int kb1 = kb0 + CHUNK_KB < kb_count ? kb0 + CHUNK_KB : kb_count;
                    for (int kb = kb0; kb < kb1; kb++) {
                        if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                        const uint32_t p_hi = sa, p_lo = sa + Cfg::kABytes, q_hi = sa + 2 * Cfg::kABytes, q_lo = q_hi + Cfg::kBBytes;
#pragma unroll
                        for (int k4 = 0; k4 < BK / UMMA_K; k4++) {
                            const uint32_t po = k4 * pf.k8_step, qo = k4 * qf.k8_step;
                            umma_tf32(tmem_d, umma_desc(pf, p_lo + po), umma_desc(qf, q_hi + qo), idesc, (kb != kb0 || k4 != 0) ? 1u : 0u);
                            umma_tf32(tmem_d, umma_desc(pf, p_hi + po), umma_desc(qf, q_lo + qo), idesc, 1u);
                            umma_tf32(tmem_d, umma_desc(pf, p_hi + po), umma_desc(qf, q_hi + qo), idesc, 1u);
                        }
                        umma_commit(empty_bar(stage));
                        if (++stage == S) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) umma_commit(acc_full_bar(buf));
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int quarter = warp & 3;           // tensor-memory lanes 32*quarter .. +31
        const int half = (warp - 4) >> 2;       // which half of the tile's columns
        uint32_t partial = 0;
        bool ok = true;
        const bool vec_ok = (prm.ldd & 3) == 0 && ((uintptr_t)prm.d & 15) == 0
                            && (!prm.second || ((uintptr_t)prm.second & 15) == 0) && (!prm.gate || ((uintptr_t)prm.gate & 15) == 0);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile / prm.tiles_n) * BM, n0 = (tile % prm.tiles_n) * BN;
            float sum[CPT];
            for (int kb0 = 0; kb0 < kb_count; kb0 += CHUNK_KB, partial++) {
                const int buf = partial & 1;
                ok = mbar_wait(acc_full_bar(buf), (partial >> 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * CPT);
                if (kb0 == 0) {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = t[i];
                    }
                } else {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = __fadd_rn(sum[s16 * 16 + i], t[i]);
                    }
                }
                tc_fence_before();
                mbar_arrive(acc_empty_bar(buf));
            }
            if (!ok) break;
            const int row = m0 + quarter * 32 + lane;
            const bool row_ok = row < prm.m;
            if (row_ok) {
#pragma unroll
                for (int g = 0; g < CPT / 4; g++) {
                    const int col = n0 + half * CPT + g * 4;
                    if ((col & ~31) < prm.n)
                        epilogue_emit4<GENERAL>(prm, row, col, sum[g * 4], sum[g * 4 + 1], sum[g * 4 + 2], sum[g * 4 + 3], vec_ok);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(prm.error_word, ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Two-SM variant (cta_group::2).  A cluster of two blocks works on one 256 x BN tile: each block
// loads its own 128 rows of P and its own half (BN / 2 rows) of Q, the even block issues one
// tcgen05.mma.cta_group::2 (M = 256) per step that reads both blocks' shared memory, and each block
// keeps the accumulator rows of its 128 result rows in its own tensor memory.  Per SM this halves
// the Q bytes that TMA writes and the tensor core reads from shared memory, which is what bounds the
// one-SM kernel (12 KB of operands per 128-clock MMA plus the refill is more than 128 B/clock).
// Partial sums are promoted to FP32 register sums exactly as in the kernel above.
// Barriers: full[s] lives in the even block and counts the bytes of both blocks' loads; empty[s] and
// acc_full[b] exist in both blocks and are signalled by two tcgen05.commit of the even block;
// acc_empty[b] lives in the even block and is signalled by the epilogue threads of both.
// ------------------------------------------------------------------------------------------------
template <int BN> struct PairConfig {
    static constexpr int kStages = BN == 256 ? 3 : 4;
    static constexpr int kABytes = BM * BK * 4;                // one plane of this block's 128 rows of P
    static constexpr int kBBytes = (BN / 2) * BK * 4;          // one plane of this block's half of Q
    static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t start = global_timer();
    for (uint32_t spin = 0;; spin++) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((spin & 63u) == 63u) {
            if (*abort_flag) return false;
            if (global_timer() - start > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
        }
    }
}
// TMA load of the two-SM form: the completion bytes may be counted on a barrier of the partner block.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void load_operand_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int kb, int r0, int mn_major) {
    if (mn_major) tma_load_3d_pair(dst, map, cluster_bar, 0, kb * BK, r0 >> 5);
    else tma_load_2d_pair(dst, map, cluster_bar, kb * BK, r0);
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

// ---- write-out of the two-SM kernel through shared memory and TMA stores ----------------------------
// An epilogue thread owns one result row, so direct stores of a warp touch 32 rows, 16 bytes each, and every
// further array written from the epilogue (a second result, the hi / lo operand planes of the result) costs as
// much again; with the FP32 promotion the write-out has two partial sums' time (about 49 000 clocks at K = 4096)
// before the tensor core waits for it.  Staged form: a warp finishes 32 columns of its 32 rows at a time in
// registers, writes them as one 128-byte-swizzled box of 32 x 32 floats to its 4 KB of shared memory and one
// lane hands the box to a TMA store, per array; the store also clips rows and columns past the matrix.
struct StoreMaps { CUtensorMap d, second, hi, lo; };

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
// Before a block leaves: its stores have completed.
__device__ __forceinline__ void staged_drain(int lane) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
}
constexpr int STAGING_BYTES = 8 * 4096;     // one box per epilogue warp

// `sum` holds the warp's CPT columns of this thread's row and is finished in place, 32 columns at a time.
// `bias_lane`: bias of columns col0 + 4 lane .. + 3 (fetched before the accumulator was waited for).
template <int CPT, bool GENERAL>
__device__ __forceinline__ void epilogue_emit_staged(const TcParams &prm, const StoreMaps &maps, uint32_t stage, int row0, int col0,
                                                     float (&sum)[CPT], float4 bias_lane, int lane) {
    const int row = row0 + lane;
    const bool row_ok = row < prm.m;
    const bool rows_left = row0 < prm.m;                            // warp-uniform
    const int width = prm.nhi ? (int)prm.nld : prm.n;               // planes carry zero padding up to their pitch
    const uint32_t mine = stage + (uint32_t)(lane * 128);
    const uint32_t twist = (uint32_t)(lane & 7);
    auto put4 = [&](int j, float a, float b, float c, float d) {     // 16-byte chunk j of this lane's row of the box
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(mine + ((((uint32_t)j) ^ twist) << 4)), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
    };
    auto reclaim = [&]() {          // the previous box has been read out of shared memory
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    };
    auto ship = [&](const CUtensorMap *map, int c0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && rows_left) {
            tma_store_2d(map, stage, c0, row0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    };
#pragma unroll
    for (int b = 0; b < CPT / 32; b++) {
        const int c0 = col0 + b * 32;
        if (c0 >= width) break;                                     // warp-uniform
        float *v = &sum[b * 32];
        float4 gate[8];
        if (prm.gate) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int col = c0 + 4 * j;
                gate[j] = (row_ok && col < prm.n) ? *reinterpret_cast<const float4 *>(prm.gate + (int64_t)row * prm.n + col) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
        reclaim();
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int col = c0 + 4 * j;
            float z[4] = {v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]};
            if (prm.bias) {
                const int src = b * 8 + j;
                z[0] = __fadd_rn(z[0], __shfl_sync(0xffffffffu, bias_lane.x, src));
                z[1] = __fadd_rn(z[1], __shfl_sync(0xffffffffu, bias_lane.y, src));
                z[2] = __fadd_rn(z[2], __shfl_sync(0xffffffffu, bias_lane.z, src));
                z[3] = __fadd_rn(z[3], __shfl_sync(0xffffffffu, bias_lane.w, src));
            }
            if (prm.gate) {
                z[0] = gate[j].x > 0.0f ? z[0] : 0.0f; z[1] = gate[j].y > 0.0f ? z[1] : 0.0f;
                z[2] = gate[j].z > 0.0f ? z[2] : 0.0f; z[3] = gate[j].w > 0.0f ? z[3] : 0.0f;
            }
            float y[4];
            if (GENERAL) {
                const float4 a = activate4(prm.act, make_float4(z[0], z[1], z[2], z[3]));
                y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) y[e] = prm.act ? relu_value(z[e]) : z[e];
            }
            if (prm.second) put4(j, z[0], z[1], z[2], z[3]);
            else put4(j, y[0], y[1], y[2], y[3]);
            const bool inside = col < prm.n;                        // n is a multiple of 4 here
#pragma unroll
            for (int e = 0; e < 4; e++) v[4 * j + e] = inside ? y[e] : 0.0f;
        }
        if (c0 < prm.n) {
            ship(&maps.d, c0);
            if (prm.second) {
                reclaim();
#pragma unroll
                for (int j = 0; j < 8; j++) put4(j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                ship(&maps.second, c0);
            }
        }
        if (prm.nhi) {
            reclaim();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float h[4], l[4];
#pragma unroll
                for (int e = 0; e < 4; e++) split_value(v[4 * j + e], h[e], l[e]);
                put4(j, h[0], h[1], h[2], h[3]);
            }
            ship(&maps.hi, c0);
            reclaim();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float h[4], l[4];
#pragma unroll
                for (int e = 0; e < 4; e++) split_value(v[4 * j + e], h[e], l[e]);
                put4(j, l[0], l[1], l[2], l[3]);
            }
            ship(&maps.lo, c0);
        }
    }
}

template <int BN, bool SLICED, bool DYNAMIC, bool GENERAL, bool STAGED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PROMOTED_THREADS, 1) gemm_tf32x3_pair_kernel(
        const __grid_constant__ CUtensorMap map_p_hi, const __grid_constant__ CUtensorMap map_p_lo,
        const __grid_constant__ CUtensorMap map_q_hi, const __grid_constant__ CUtensorMap map_q_lo,
        const __grid_constant__ StoreMaps stores, TcParams prm, SliceParams slc) {
    static_assert(!(STAGED && SLICED), "a slice writes its raw partial product directly");
    using Cfg = PairConfig<BN>;
    constexpr int S = Cfg::kStages;
    constexpr int CPT = BN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S * Cfg::kStageBytes + (STAGED ? STAGING_BYTES : 0));
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) accumulator full, [2S+2..2S+4) accumulator empty,
    // [2S+4..2S+4+R) unit published, [2S+4+R..2S+4+2R) unit slot free (used in the even block)
    constexpr int R = 4;                    // depth of the ring of published unit numbers
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 4 + 2 * R);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile int *sched_unit = reinterpret_cast<volatile int *>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };
    auto sched_full_bar = [&](int r) { return bar_base + 8u * (2 * S + 4 + r); };
    auto sched_empty_bar = [&](int r) { return bar_base + 8u * (2 * S + 4 + R + r); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 512); }
        // a published unit is consumed by the issuer, the partner's producer and one lane of each of
        // the 16 epilogue warps of the pair
        for (int r = 0; r < R; r++) { mbar_init(sched_full_bar(r), 1); mbar_init(sched_empty_bar(r), 18); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {        // the same warp of both blocks allocates the pair's tensor memory together
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();     // the partner's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = prm.tiles_m * prm.tiles_n;      // tiles of 256 x BN
    const int kb_count = prm.k_blocks;
    // a unit is one tile over one slice of the contraction; without slicing a unit is a tile and the
    // slice arithmetic below folds away at compile time
    const int total_units = SLICED ? total_tiles * slc.slices : total_tiles;
    const int kb_per_slice = SLICED ? slc.kb_per_slice : kb_count;
    const int CHUNK_KB = prm.chunk_kb;
    const uint32_t smem_base = smem_u32(smem);
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    // Dynamic unit assignment (DYNAMIC): the even block's producer thread takes the next unit number from
    // a counter in global memory and publishes it to both blocks through a ring of R slots; every other
    // role reads the ring in the same order.  A pair that starts late, because another kernel (an
    // all-reduce) held its SMs, then simply takes fewer units, where a fixed assignment would make the
    // whole product wait for it.  -1 ends the sequence; a wait that gives up also returns -1.
    auto sched_publish = [&](int seq) -> int {          // even block, producer thread only
        const int r = seq % R;
        if (!mbar_wait_cluster(sched_empty_bar(r), (((uint32_t)seq / R) & 1u) ^ 1u, abort_flag)) return -1;
        int u = atomicAdd(slc.unit_counter, 1);
        if (u >= total_units) u = -1;
        sched_unit[r] = u;
        asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(map_to_rank(smem_u32((const void *)(sched_unit + r)), 1)), "r"(u) : "memory");
        mbar_arrive_cluster(map_to_rank(sched_full_bar(r), 0));
        mbar_arrive_cluster(map_to_rank(sched_full_bar(r), 1));
        return u;
    };
    auto sched_take = [&](int seq, bool arrive) -> int { // every other role; `arrive` from one lane per warp
        const int r = seq % R;
        if (!mbar_wait_cluster(sched_full_bar(r), ((uint32_t)seq / R) & 1u, abort_flag)) return -1;
        const int u = sched_unit[r];
        if (arrive) mbar_arrive_cluster(map_to_rank(sched_empty_bar(r), 0));
        return u;
    };

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            int seq = 0;
            int unit = !DYNAMIC ? pair : (rank == 0 ? sched_publish(seq) : sched_take(seq, true));
            for (; unit >= 0 && unit < total_units && ok; ) {
                // the next unit number is requested before this unit's loads, so the counter's latency hides
                int next = unit + pairs;
                if (DYNAMIC && rank == 0) next = sched_publish(++seq);
                const int tile = SLICED ? unit % total_tiles : unit, slice = SLICED ? unit / total_tiles : 0;
                int mi, ni;
                tile_origin(tile, prm.tiles_m, prm.tiles_n, slc.group_n, mi, ni);
                const int m0 = mi * (2 * BM) + (int)rank * BM;
                const int n0 = ni * BN + (int)rank * (BN / 2);
                const int kb_first = slice * kb_per_slice;
                const int kb_last = (SLICED && kb_first + kb_per_slice < kb_count) ? kb_first + kb_per_slice : kb_count;
                for (int kb = kb_first; kb < kb_last; kb++) {
                    if (!mbar_wait_cluster(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                    const uint32_t leader_full = map_to_rank(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * Cfg::kStageBytes);
                    load_operand_pair(sa, &map_p_hi, leader_full, kb, m0, prm.p_mn);
                    load_operand_pair(sa + Cfg::kABytes, &map_p_lo, leader_full, kb, m0, prm.p_mn);
                    load_operand_pair(sa + 2 * Cfg::kABytes, &map_q_hi, leader_full, kb, n0, prm.q_mn);
                    load_operand_pair(sa + 2 * Cfg::kABytes + Cfg::kBBytes, &map_q_lo, leader_full, kb, n0, prm.q_mn);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
                if (DYNAMIC && rank != 0) next = sched_take(++seq, true);
                unit = next;
            }
        }
    } else if (warp == 1 && rank == 0) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(2 * BM, BN, prm.p_mn, prm.q_mn);
            const OperandForm pf = operand_form(prm.p_mn), qf = operand_form(prm.q_mn);
            int stage = 0; uint32_t phase = 0;
            uint32_t partial = 0;
            bool ok = true;
            int seq = 0;
            for (int unit = DYNAMIC ? sched_take(seq, true) : pair; unit >= 0 && unit < total_units && ok;
                 unit = DYNAMIC ? sched_take(++seq, true) : unit + pairs) {
                const int kb_first = SLICED ? (unit / total_tiles) * kb_per_slice : 0;
                const int kb_last = (SLICED && kb_first + kb_per_slice < kb_count) ? kb_first + kb_per_slice : kb_count;
                for (int kb0 = kb_first; kb0 < kb_last && ok; kb0 += CHUNK_KB, partial++) {
                    const int buf = partial & 1;
                    if (!mbar_wait_cluster(acc_empty_bar(buf), ((partial >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                    const int kb1 = kb0 + CHUNK_KB < kb_last ? kb0 + CHUNK_KB : kb_last;
                    for (int kb = kb0; kb < kb1; kb++) {
                        if (!mbar_wait_cluster(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                        const uint32_t p_hi = sa, p_lo = sa + Cfg::kABytes, q_hi = sa + 2 * Cfg::kABytes, q_lo = q_hi + Cfg::kBBytes;
#pragma unroll
                        for (int k4 = 0; k4 < BK / UMMA_K; k4++) {
                            const uint32_t po = k4 * pf.k8_step, qo = k4 * qf.k8_step;
                            umma_tf32_pair(tmem_d, umma_desc(pf, p_lo + po), umma_desc(qf, q_hi + qo), idesc, (kb != kb0 || k4 != 0) ? 1u : 0u);
                            umma_tf32_pair(tmem_d, umma_desc(pf, p_hi + po), umma_desc(qf, q_lo + qo), idesc, 1u);
                            umma_tf32_pair(tmem_d, umma_desc(pf, p_hi + po), umma_desc(qf, q_hi + qo), idesc, 1u);
                        }
                        umma_commit_pair(empty_bar(stage));                      // this block's producer
                        umma_commit_pair(map_to_rank(empty_bar(stage), 1));      // the partner's producer
                        if (++stage == S) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) {
                        umma_commit_pair(acc_full_bar(buf));
                        umma_commit_pair(map_to_rank(acc_full_bar(buf), 1));
                    }
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int quarter = warp & 3;
        const int half = (warp - 4) >> 2;
        uint32_t partial = 0;
        bool ok = true;
        const bool vec_ok = (prm.ldd & 3) == 0 && ((uintptr_t)prm.d & 15) == 0
                            && (!prm.second || ((uintptr_t)prm.second & 15) == 0) && (!prm.gate || ((uintptr_t)prm.gate & 15) == 0);
        int seq = 0;
        // lane 0 alone reads the ring (it frees the slot at once, so no other lane may look at it)
        auto warp_take = [&](int sequence) -> int {
            int u = 0;
            if (lane == 0) u = sched_take(sequence, true);
            return __shfl_sync(0xffffffffu, u, 0);
        };
        for (int unit = DYNAMIC ? warp_take(seq) : pair; unit >= 0 && unit < total_units && ok;
             unit = DYNAMIC ? warp_take(++seq) : unit + pairs) {
            const int tile = SLICED ? unit % total_tiles : unit, slice = SLICED ? unit / total_tiles : 0;
            int mi, ni;
            tile_origin(tile, prm.tiles_m, prm.tiles_n, slc.group_n, mi, ni);
            const int m0 = mi * (2 * BM) + (int)rank * BM, n0 = ni * BN;
            const int kb_first = slice * kb_per_slice;
            const int kb_last = (SLICED && kb_first + kb_per_slice < kb_count) ? kb_first + kb_per_slice : kb_count;
            float4 bias_lane = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if constexpr (STAGED) {
                const int bias_col = n0 + half * CPT + lane * 4;
                if (prm.bias && bias_col < prm.n) bias_lane = *reinterpret_cast<const float4 *>(prm.bias + bias_col);
            }
            float sum[CPT];
            for (int kb0 = kb_first; kb0 < kb_last; kb0 += CHUNK_KB, partial++) {
                const int buf = partial & 1;
                ok = mbar_wait_cluster(acc_full_bar(buf), (partial >> 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * CPT);
                if (kb0 == kb_first) {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = t[i];
                    }
                } else {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = __fadd_rn(sum[s16 * 16 + i], t[i]);
                    }
                }
                tc_fence_before();
                mbar_arrive_cluster(map_to_rank(acc_empty_bar(buf), 0));
            }
            if (!ok) break;
            if constexpr (STAGED) {
                epilogue_emit_staged<CPT, GENERAL>(prm, stores, smem_base + (uint32_t)(S * Cfg::kStageBytes + (warp - 4) * 4096),
                                                   m0 + quarter * 32, n0 + half * CPT, sum, bias_lane, lane);
                continue;
            }
            const int row = m0 + quarter * 32 + lane;
            const bool row_ok = row < prm.m;
            if constexpr (SLICED) {
                // a slice of a split contraction writes its raw partial product to the workspace
                // ([slice][m][slice_ld]; the launch guarantees there is no other epilogue work then);
                // slice_combine_kernel adds the slices in a fixed order
                if (row_ok) {
                    float *wrow = slc.ws + ((int64_t)slice * prm.m + row) * slc.ld;
#pragma unroll
                    for (int g = 0; g < CPT / 4; g++) {
                        const int col = n0 + half * CPT + g * 4;
                        if (col < slc.ld)
                            *reinterpret_cast<float4 *>(wrow + col) = make_float4(sum[g * 4], sum[g * 4 + 1], sum[g * 4 + 2], sum[g * 4 + 3]);
                    }
                }
            } else if (row_ok) {
#pragma unroll
                for (int g = 0; g < CPT / 4; g++) {
                    const int col = n0 + half * CPT + g * 4;
                    if ((col & ~31) < prm.n)
                        epilogue_emit4<GENERAL>(prm, row, col, sum[g * 4], sum[g * 4 + 1], sum[g * 4 + 2], sum[g * 4 + 3], vec_ok);
                }
            }
        }
        if constexpr (STAGED) staged_drain(lane);
    }

    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();     // neither block frees tensor memory or leaves while the partner may still signal it
    if (threadIdx.x == 0 && *abort_flag) atomicOr(prm.error_word, ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

// Adds the slices of a split contraction in ascending order, one binary32 rounding per addition.
__global__ void slice_combine_kernel(const float *__restrict__ ws, int slices, int64_t m, int64_t n, int64_t slice_ld, float *d, int64_t ldd) {
    const int64_t quads = slice_ld >> 2, total = m * quads;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / quads, c = (i - r * quads) << 2;
        float4 acc = *reinterpret_cast<const float4 *>(ws + r * slice_ld + c);
        for (int sl = 1; sl < slices; sl++) {
            const float4 v = *reinterpret_cast<const float4 *>(ws + ((int64_t)sl * m + r) * slice_ld + c);
            acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
        }
        float *out = d + r * ldd + c;
        if (c + 3 < n && (ldd & 3) == 0 && ((uintptr_t)d & 15) == 0) *reinterpret_cast<float4 *>(out) = acc;
        else { const float v[4] = {acc.x, acc.y, acc.z, acc.w}; for (int e = 0; e < 4; e++) if (c + e < n) out[e] = v[e]; }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D map over a K-major [rows, kp] FP32 plane: box = 32 floats (one 128-byte swizzle row) x box_rows.
bool make_plane_map(CUtensorMap *map, const float *plane, int64_t rows, int64_t kp, int64_t pitch, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)kp, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 4};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)plane, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// 3-D map over an MN-major [k, rows_padded] plane, seen as (32 rows, k, rows_padded / 32): one box of
// (32, 32, box_rows / 32) lands in shared memory as box_rows / 32 consecutive [32 k][128 byte] slabs
// in the 32-byte-atom swizzle, which is the MN-major operand layout.  Contraction steps past k read as zero.
bool make_plane_map_mn(CUtensorMap *map, const float *plane, int64_t k, int64_t rows_padded, int64_t pitch, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {32, (cuuint64_t)k, (cuuint64_t)(rows_padded / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)pitch * 4, 128};
    cuuint32_t box[3] = {32, (cuuint32_t)BK, (cuuint32_t)(box_rows / 32)};
    cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void *)plane, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


// ------------------------------------------------------------------------------------------------
// 16-bit storage (BFLOAT16 / FLOAT16) with a FLOAT32 working type.
//
//  * gemm_exact_low_kernel: the exact CUDA-core product on 16-bit operands: every cell is the reference's
//    ascending-k FLOAT32 chain over the widened operands and one narrowing of the sum
//    (CpuMatmulReferenceKernel.java:71-93), then ADD of the bias and the activation, each narrowed once.
//  * gemm_low_kernel: the tensor-core product.  16-bit values need no hi / lo split: TMA loads the operand
//    tiles straight from the matrices themselves (K-major, 64 elements = one 128-byte swizzle row per
//    k-block) and one tcgen05.mma kind::f16 per 16 contraction steps accumulates in FP32 in tensor memory.
//    Partial sums are promoted to round-to-nearest FP32 register sums exactly as in the 3xTF32 kernels
//    (the tensor core's own accumulation truncates).  Same warp roles and barriers as
//    gemm_tf32x3_promoted_kernel.
// ------------------------------------------------------------------------------------------------
struct LowEpilogue {
    const uint16_t *bias;       // [n] storage bits, or null
    int act;                    // activation wire code, 0 none
    uint16_t *second;           // dense [m,n]: when set, `out` receives z and `second` act(z)
};

template <int KIND>
__device__ __forceinline__ void low_finish(float sum, const LowEpilogue &ep, int64_t col, float &z_out, float &y_out) {
    float z = low_round<KIND>(sum);                                                // MATMUL's own narrowing
    if (ep.bias) z = low_round<KIND>(__fadd_rn(z, low_decode<KIND>(ep.bias[col])));   // ADD
    z_out = z;
    y_out = ep.act ? low_round<KIND>(low_activation_value(ep.act, z)) : z;          // activation
}

template <int KIND>
__global__ void __launch_bounds__(256) gemm_exact_low_kernel(int64_t m, int64_t n, int64_t k,
        const uint16_t *__restrict__ a, int64_t a_ms, int64_t a_ks, const uint16_t *__restrict__ b, int64_t b_ks, int64_t b_ns,
        uint16_t *c, int64_t c_ms, int64_t c_ns, LowEpilogue ep) {
    __shared__ float as[XK][XT + 4];
    __shared__ float bs[XK][XT + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * XT, n0 = (int64_t)blockIdx.x * XT;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    const bool a_kfast = a_ks == 1, b_nfast = b_ns == 1;
    for (int64_t k0 = 0; k0 < k; k0 += XK) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            int e = tid + q * 256;
            int row = a_kfast ? e / XK : e % XT, kk = a_kfast ? e % XK : e / XT;
            int64_t gm = m0 + row, gk = k0 + kk;
            as[kk][row] = (gm < m && gk < k) ? low_decode<KIND>(a[gm * a_ms + gk * a_ks]) : 0.0f;
            int col = b_nfast ? e % XT : e / XK, kb = b_nfast ? e / XT : e % XK;
            int64_t gn = n0 + col, gkb = k0 + kb;
            bs[kb][col] = (gn < n && gkb < k) ? low_decode<KIND>(b[gkb * b_ks + gn * b_ns]) : 0.0f;
        }
        __syncthreads();
        const int depth = (int)((k - k0) < XK ? (k - k0) : XK);
        if (k == 1) {
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __fmul_rn(as[0][ty * 4 + i], bs[0][tx * 4 + j]);
        } else {
            for (int kk = 0; kk < depth; kk++) {
                float av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) av[i] = as[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; j++) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int64_t gm = m0 + ty * 4 + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int64_t gn = n0 + tx * 4 + j;
            if (gn >= n) continue;
            float z, y;
            low_finish<KIND>(acc[i][j], ep, gn, z, y);
            if (ep.second) { c[gm * c_ms + gn * c_ns] = low_encode<KIND>(z); ep.second[gm * n + gn] = low_encode<KIND>(y); }
            else c[gm * c_ms + gn * c_ns] = low_encode<KIND>(y);
        }
    }
}

constexpr int LOW_BK = 64;              // 16-bit elements per k-block: one 128-byte swizzle row
constexpr int LOW_UMMA_K = 16;          // kind::f16 contracts 16 elements (32 bytes) per instruction

template <int BN> struct LowConfig {
    static constexpr int kABytes = BM * 128;                // 128 rows of one k-block
    static constexpr int kBBytes = BN * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStagingBytes = BN >= 128 ? 8 * 4096 : 0;      // one box of 32 rows x 64 columns per epilogue warp
    static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

struct LowParams {
    uint16_t *d; int64_t ldd;
    int m, n, k_blocks;
    int tiles_m, tiles_n;
    int chunk_kb;
    LowEpilogue ep;
    int *error_word;
    int staged;         // results leave through shared memory and TMA stores (see low_emit_staged)
};

// Instruction descriptor of kind::f16: FP32 accumulate, both operands BF16 (format 1) or F16 (format 0), K-major.
__device__ __forceinline__ uint32_t umma_idesc_low(int rows, int bn, int kind) {
    const uint32_t format = kind == 1 ? 1u : 0u;
    return (1u << 4) | (format << 7) | (format << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(rows >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// The elementary functions of the activations, out of line (see activate4).
template <int KIND>
__device__ __noinline__ float4 low_activate4(int act, float4 z) {
    return make_float4(low_round<KIND>(low_activation_value(act, z.x)), low_round<KIND>(low_activation_value(act, z.y)),
                       low_round<KIND>(low_activation_value(act, z.z)), low_round<KIND>(low_activation_value(act, z.w)));
}

// Four adjacent result cells of one row: narrow the sum, add the bias and narrow, apply the activation and
// narrow, store 8 bytes (and the pre-activation beside it when asked).
template <int KIND>
__device__ __forceinline__ void low_emit4(const LowParams &prm, int row, int col, float s0, float s1, float s2, float s3, bool vec_ok) {
    float z[4] = {low_round<KIND>(s0), low_round<KIND>(s1), low_round<KIND>(s2), low_round<KIND>(s3)};
    const bool full = col + 3 < prm.n;
    if (prm.ep.bias) {
        if (full && vec_ok) {
            const uint2 raw = *reinterpret_cast<const uint2 *>(prm.ep.bias + col);
            const uint16_t bits[4] = {(uint16_t)(raw.x & 0xffffu), (uint16_t)(raw.x >> 16), (uint16_t)(raw.y & 0xffffu), (uint16_t)(raw.y >> 16)};
#pragma unroll
            for (int e = 0; e < 4; e++) z[e] = low_round<KIND>(__fadd_rn(z[e], low_decode<KIND>(bits[e])));
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) if (col + e < prm.n) z[e] = low_round<KIND>(__fadd_rn(z[e], low_decode<KIND>(prm.ep.bias[col + e])));
        }
    }
    float y[4] = {z[0], z[1], z[2], z[3]};
    if (prm.ep.act == (int)Op::RELU) {
#pragma unroll
        for (int e = 0; e < 4; e++) y[e] = relu_value(z[e]);            // exact on a storage value: no second narrowing needed
    } else if (prm.ep.act) {
        const float4 a = low_activate4<KIND>(prm.ep.act, make_float4(z[0], z[1], z[2], z[3]));
        y[0] = a.x; y[1] = a.y; y[2] = a.z; y[3] = a.w;
    }
    uint16_t *drow = prm.d + (int64_t)row * prm.ldd;
    uint16_t *srow = prm.ep.second ? prm.ep.second + (int64_t)row * prm.n : nullptr;
    auto pack = [](const float (&v)[4]) {
        return make_uint2((uint32_t)low_encode<KIND>(v[0]) | ((uint32_t)low_encode<KIND>(v[1]) << 16),
                          (uint32_t)low_encode<KIND>(v[2]) | ((uint32_t)low_encode<KIND>(v[3]) << 16));
    };
    if (full && vec_ok) {
        if (srow) { *reinterpret_cast<uint2 *>(drow + col) = pack(z); *reinterpret_cast<uint2 *>(srow + col) = pack(y); }
        else *reinterpret_cast<uint2 *>(drow + col) = pack(y);
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (col + e >= prm.n) continue;
            if (srow) { drow[col + e] = low_encode<KIND>(z[e]); srow[col + e] = low_encode<KIND>(y[e]); }
            else drow[col + e] = low_encode<KIND>(y[e]);
        }
    }
}

// ---- write-out through shared memory ------------------------------------------------------------
// An epilogue thread owns one result row (tensor-memory lane = row), so direct stores of a warp go to 32
// different rows, 8 bytes each: measured on 8192 x 4096 x 4096 BF16 the write-out of a tile then takes
// twice as long as the tile's MMAs (tensor pipe 53-58 % active; with the write-out switched off the same
// launch ran 1.5x faster).  Staged form: every warp converts its 32 rows x CPT columns with packed
// conversions into 128-byte-swizzled boxes of 32 rows x 64 columns in shared memory and one lane hands each
// box to a TMA store, which also clips rows and columns past the matrix.  Same arithmetic, node by node, as
// low_emit4: narrow the sum; add the bias in FLOAT32 and narrow; activation and narrow.
template <int KIND> __device__ __forceinline__ uint32_t low_pack2(float lo, float hi) {
    uint32_t r;
    if constexpr (KIND == 1) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
template <int KIND> __device__ __forceinline__ void low_unpack2(uint32_t r, float &lo, float &hi) {
    if constexpr (KIND == 1) { lo = __uint_as_float(r << 16); hi = __uint_as_float(r & 0xffff0000u); }
    else { lo = __half2float(__ushort_as_half((uint16_t)(r & 0xffffu))); hi = __half2float(__ushort_as_half((uint16_t)(r >> 16))); }
}
// Math.max(x, +0) on both halves: NaN stays NaN, -0 and negatives give +0.
template <int KIND> __device__ __forceinline__ uint32_t low_relu2(uint32_t r) {
    uint32_t d;
    if constexpr (KIND == 1) asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(r), "r"(0u));
    else asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(d) : "r"(r), "r"(0u));
    return d;
}
// The packed instructions give every NaN as 0x7FFF; the storage types' NaN is 0x7FC0 / 0x7E00 (low_encode).
template <int KIND> __device__ __forceinline__ uint32_t low_canonical_nan2(uint32_t r) {
    constexpr uint32_t inf2 = KIND == 1 ? 0x7F807F80u : 0x7C007C00u, nan2 = KIND == 1 ? 0x7FC07FC0u : 0x7E007E00u;
    const uint32_t mask = __vcmpgtu2(r & 0x7FFF7FFFu, inf2);
    return mask ? ((r & ~mask) | (nan2 & mask)) : r;
}

// The bias of a warp's columns lives in its lanes' registers, four columns per lane (lane l: columns
// 4 l .. 4 l + 3 of the warp's first 128), fetched before the warp waits for the accumulator: a load from
// global memory between the stores of the write-out would cost a round trip to L2 per eight columns.
__device__ __forceinline__ uint2 low_bias_lane(const LowParams &prm, int col) {
    uint2 b = make_uint2(0u, 0u);
    if (!prm.ep.bias || col >= prm.n) return b;
    if (col + 3 < prm.n && ((uintptr_t)(prm.ep.bias + col) & 7) == 0) return *reinterpret_cast<const uint2 *>(prm.ep.bias + col);
#pragma unroll
    for (int e = 0; e < 4; e++)
        if (col + e < prm.n) (e < 2 ? b.x : b.y) |= (uint32_t)prm.ep.bias[col + e] << (16 * (e & 1));
    return b;
}

// Eight adjacent result cells of one row as four packed words; `group` is their index among the warp's
// groups of eight columns (the bias of group g is in lanes 2 g and 2 g + 1).
template <int KIND>
__device__ __forceinline__ uint4 low_finish8(const LowParams &prm, int group, const float *s, uint2 bias_lane) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; e++) w[e] = low_pack2<KIND>(s[2 * e], s[2 * e + 1]);            // MATMUL's own narrowing
    if (prm.ep.bias) {
        uint32_t b[4];
        b[0] = __shfl_sync(0xffffffffu, bias_lane.x, 2 * group);
        b[1] = __shfl_sync(0xffffffffu, bias_lane.y, 2 * group);
        b[2] = __shfl_sync(0xffffffffu, bias_lane.x, 2 * group + 1);
        b[3] = __shfl_sync(0xffffffffu, bias_lane.y, 2 * group + 1);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float z0, z1, b0, b1;
            low_unpack2<KIND>(w[e], z0, z1);
            low_unpack2<KIND>(b[e], b0, b1);
            w[e] = low_pack2<KIND>(__fadd_rn(z0, b0), __fadd_rn(z1, b1));                 // ADD
        }
    }
    if (prm.ep.act == (int)Op::RELU) {
#pragma unroll
        for (int e = 0; e < 4; e++) w[e] = low_relu2<KIND>(w[e]);
    } else if (prm.ep.act) {
        float z[8];
#pragma unroll
        for (int e = 0; e < 4; e++) low_unpack2<KIND>(w[e], z[2 * e], z[2 * e + 1]);
        const float4 a0 = low_activate4<KIND>(prm.ep.act, make_float4(z[0], z[1], z[2], z[3]));
        const float4 a1 = low_activate4<KIND>(prm.ep.act, make_float4(z[4], z[5], z[6], z[7]));
        w[0] = low_pack2<KIND>(a0.x, a0.y); w[1] = low_pack2<KIND>(a0.z, a0.w);
        w[2] = low_pack2<KIND>(a1.x, a1.y); w[3] = low_pack2<KIND>(a1.z, a1.w);
    }
#pragma unroll
    for (int e = 0; e < 4; e++) w[e] = low_canonical_nan2<KIND>(w[e]);
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// One warp's 32 rows x CPT columns of a finished tile, 64 columns at a time.  `stage` is this warp's 4 KB of
// shared memory (1024-byte aligned): one box of 32 rows x 128 bytes, 16-byte chunk j of row r at chunk
// j ^ (r & 7) as the 128-byte swizzle of the store's tensor map expects (and conflict-free for a thread per row).
// One box per warp rather than one per 64 columns: the shared memory saved is one more stage of operands, and
// the main loop is bound by how many operand bytes are in flight (see LowPairConfig).
template <int KIND, int CPT>
__device__ __forceinline__ void low_emit_staged(const LowParams &prm, const CUtensorMap *map_d, uint32_t stage, int row0, int col0,
                                                const float (&sum)[CPT], uint2 bias_lane, int lane) {
    static_assert(CPT % 64 == 0 && CPT <= 128, "boxes of 64 columns; the bias registers cover 128");
#pragma unroll
    for (int b = 0; b < CPT / 64; b++) {
        if (col0 + b * 64 >= prm.n) break;          // warp-uniform
        // the previous box has been read out of shared memory
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint4 words = low_finish8<KIND>(prm, b * 8 + j, &sum[b * 64 + j * 8], bias_lane);
            const uint32_t dst = stage + (uint32_t)(lane * 128 + ((j ^ (lane & 7)) << 4));
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(words.x), "r"(words.y), "r"(words.z), "r"(words.w) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && row0 < prm.m) {
            tma_store_2d(map_d, stage, col0 + b * 64, row0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
}

template <int BN, int KIND>
__global__ void __launch_bounds__(PROMOTED_THREADS, 1) gemm_low_kernel(
        const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_d,
        LowParams prm) {
    using Cfg = LowConfig<BN>;
    constexpr int S = Cfg::kStages;
    constexpr int CPT = BN / 2;             // result columns per epilogue thread
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S * Cfg::kStageBytes + Cfg::kStagingBytes);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) accumulator full, [2S+2..2S+4) accumulator empty
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 256); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = prm.tiles_m * prm.tiles_n;
    const int kb_count = prm.k_blocks;
    const int CHUNK_KB = prm.chunk_kb;
    const uint32_t smem_base = smem_u32(smem);

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            uint32_t armed_phase[S]; bool armed[S];
            for (int s = 0; s < S; s++) { armed[s] = false; armed_phase[s] = 0; }
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / prm.tiles_n) * BM, n0 = (tile % prm.tiles_n) * BN;
                for (int kb = 0; kb < kb_count; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                    mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    armed[stage] = true; armed_phase[stage] = phase;
                    // element coordinate kb * 64: 128 bytes, always a multiple of 16; rows and columns past the
                    // matrix read as zeros
                    tma_load_2d(sa, &map_p, full_bar(stage), kb * LOW_BK, m0);
                    tma_load_2d(sa + Cfg::kABytes, &map_q, full_bar(stage), kb * LOW_BK, n0);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok || *abort_flag) {
                for (int s = 0; s < S; s++) if (armed[s]) mbar_wait(full_bar(s), armed_phase[s], abort_flag);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_low(BM, BN, KIND);
            const OperandForm form = operand_form(0);       // K-major, 128-byte swizzle: 32 bytes per MMA step
            int stage = 0; uint32_t phase = 0;
            uint32_t partial = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                for (int kb0 = 0; kb0 < kb_count && ok; kb0 += CHUNK_KB, partial++) {
                    const int buf = partial & 1;
                    if (!mbar_wait(acc_empty_bar(buf), ((partial >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                    const int kb1 = kb0 + CHUNK_KB < kb_count ? kb0 + CHUNK_KB : kb_count;
                    for (int kb = kb0; kb < kb1; kb++) {
                        if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t pa = smem_base + stage * Cfg::kStageBytes, qa = pa + Cfg::kABytes;
#pragma unroll
                        for (int k4 = 0; k4 < LOW_BK / LOW_UMMA_K; k4++) {
                            const uint32_t step = k4 * form.k8_step;
                            umma_f16(tmem_d, umma_desc(form, pa + step), umma_desc(form, qa + step), idesc, (kb != kb0 || k4 != 0) ? 1u : 0u);
                        }
                        umma_commit(empty_bar(stage));
                        if (++stage == S) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) umma_commit(acc_full_bar(buf));
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int quarter = warp & 3;           // tensor-memory lanes 32*quarter .. +31
        const int half = (warp - 4) >> 2;       // which half of the tile's columns
        uint32_t partial = 0;
        bool ok = true;
        const bool vec_ok = (prm.ldd & 3) == 0 && ((uintptr_t)prm.d & 7) == 0 && (prm.n & 3) == 0
                            && (!prm.ep.second || ((uintptr_t)prm.ep.second & 7) == 0) && (!prm.ep.bias || ((uintptr_t)prm.ep.bias & 7) == 0);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile / prm.tiles_n) * BM, n0 = (tile % prm.tiles_n) * BN;
            const uint2 bias_lane = prm.staged ? low_bias_lane(prm, n0 + half * CPT + lane * 4) : make_uint2(0u, 0u);
            float sum[CPT];
            for (int kb0 = 0; kb0 < kb_count; kb0 += CHUNK_KB, partial++) {
                const int buf = partial & 1;
                ok = mbar_wait(acc_full_bar(buf), (partial >> 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * CPT);
                if (kb0 == 0) {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = t[i];
                    }
                } else {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = __fadd_rn(sum[s16 * 16 + i], t[i]);
                    }
                }
                tc_fence_before();
                mbar_arrive(acc_empty_bar(buf));
            }
            if (!ok) break;
            if constexpr (CPT >= 64) {
                if (prm.staged) {
                    low_emit_staged<KIND, CPT>(prm, &map_d, smem_base + (uint32_t)(S * Cfg::kStageBytes + (warp - 4) * 4096),
                                               m0 + quarter * 32, n0 + half * CPT, sum, bias_lane, lane);
                    continue;
                }
            }
            const int row = m0 + quarter * 32 + lane;
            if (row < prm.m) {
#pragma unroll
                for (int g = 0; g < CPT / 4; g++) {
                    const int col = n0 + half * CPT + g * 4;
                    if (col < prm.n) low_emit4<KIND>(prm, row, col, sum[g * 4], sum[g * 4 + 1], sum[g * 4 + 2], sum[g * 4 + 3], vec_ok);
                }
            }
        }
        if (prm.staged) staged_drain(lane);
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(prm.error_word, ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}


// Two-SM form of the 16-bit product (cta_group::2, M = 256, tiles of 256 x 256).  Each block of the pair loads
// its 128 rows of P and its 128 of the tile's 256 rows of Q, so one stage is 32 KB per block and six stages
// fit beside the write-out boxes; the even block issues the MMAs for both.  A k-block of 64 elements is 512
// clocks of MMA, a third of the FP32 kernel's, so the operand bytes in flight, not a bandwidth, bound the
// main loop: with five stages ncu showed the tensor pipe active in 73 % of the cycles while L1, L2 and DRAM
// were below half of their peaks.  Roles, barriers and tile order are those of the two-SM FP32 kernel above;
// tiles are assigned to pairs in fixed rotation.
struct LowPairConfig {
    static constexpr int BN = 256;
    static constexpr int kStages = 6;
    static constexpr int kABytes = BM * 128;
    static constexpr int kBBytes = (BN / 2) * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStagingBytes = 8 * 4096;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
};

__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PROMOTED_THREADS, 1) gemm_low_pair_kernel(
        const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_d,
        LowParams prm, int group_n) {
    using Cfg = LowPairConfig;
    constexpr int BN = Cfg::BN;
    constexpr int S = Cfg::kStages;
    constexpr int CPT = BN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S * Cfg::kStageBytes + Cfg::kStagingBytes);
    // bars[0..S) full (even block), [S..2S) empty, [2S..2S+2) accumulator full, [2S+2..2S+4) accumulator empty (even block)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * S + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 512); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = prm.tiles_m * prm.tiles_n;      // tiles of 256 x 256
    const int kb_count = prm.k_blocks;
    const int CHUNK_KB = prm.chunk_kb;
    const uint32_t smem_base = smem_u32(smem);
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
                int mi, ni;
                tile_origin(tile, prm.tiles_m, prm.tiles_n, group_n, mi, ni);
                const int m0 = mi * (2 * BM) + (int)rank * BM;
                const int n0 = ni * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < kb_count; kb++) {
                    if (!mbar_wait_cluster(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
                    const uint32_t leader_full = map_to_rank(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * Cfg::kStageBytes);
                    tma_load_2d_pair(sa, &map_p, leader_full, kb * LOW_BK, m0);
                    tma_load_2d_pair(sa + Cfg::kABytes, &map_q, leader_full, kb * LOW_BK, n0);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1 && rank == 0) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_low(2 * BM, BN, KIND);
            const OperandForm form = operand_form(0);
            int stage = 0; uint32_t phase = 0;
            uint32_t partial = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
                for (int kb0 = 0; kb0 < kb_count && ok; kb0 += CHUNK_KB, partial++) {
                    const int buf = partial & 1;
                    if (!mbar_wait_cluster(acc_empty_bar(buf), ((partial >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                    const int kb1 = kb0 + CHUNK_KB < kb_count ? kb0 + CHUNK_KB : kb_count;
                    for (int kb = kb0; kb < kb1; kb++) {
                        if (!mbar_wait_cluster(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t pa = smem_base + stage * Cfg::kStageBytes, qa = pa + Cfg::kABytes;
#pragma unroll
                        for (int k4 = 0; k4 < LOW_BK / LOW_UMMA_K; k4++) {
                            const uint32_t step = k4 * form.k8_step;
                            umma_f16_pair(tmem_d, umma_desc(form, pa + step), umma_desc(form, qa + step), idesc, (kb != kb0 || k4 != 0) ? 1u : 0u);
                        }
                        umma_commit_pair(empty_bar(stage));
                        umma_commit_pair(map_to_rank(empty_bar(stage), 1));
                        if (++stage == S) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) {
                        umma_commit_pair(acc_full_bar(buf));
                        umma_commit_pair(map_to_rank(acc_full_bar(buf), 1));
                    }
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int quarter = warp & 3;
        const int half = (warp - 4) >> 2;
        uint32_t partial = 0;
        bool ok = true;
        const bool vec_ok = (prm.ldd & 3) == 0 && ((uintptr_t)prm.d & 7) == 0 && (prm.n & 3) == 0
                            && (!prm.ep.second || ((uintptr_t)prm.ep.second & 7) == 0) && (!prm.ep.bias || ((uintptr_t)prm.ep.bias & 7) == 0);
        for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
            int mi, ni;
            tile_origin(tile, prm.tiles_m, prm.tiles_n, group_n, mi, ni);
            const int m0 = mi * (2 * BM) + (int)rank * BM, n0 = ni * BN;
            const uint2 bias_lane = prm.staged ? low_bias_lane(prm, n0 + half * CPT + lane * 4) : make_uint2(0u, 0u);
            float sum[CPT];
            for (int kb0 = 0; kb0 < kb_count; kb0 += CHUNK_KB, partial++) {
                const int buf = partial & 1;
                ok = mbar_wait_cluster(acc_full_bar(buf), (partial >> 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * CPT);
                if (kb0 == 0) {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = t[i];
                    }
                } else {
#pragma unroll
                    for (int s16 = 0; s16 < CPT / 16; s16++) {
                        float t[16];
                        tmem_load16(taddr + (uint32_t)(s16 * 16), t);
#pragma unroll
                        for (int i = 0; i < 16; i++) sum[s16 * 16 + i] = __fadd_rn(sum[s16 * 16 + i], t[i]);
                    }
                }
                tc_fence_before();
                mbar_arrive_cluster(map_to_rank(acc_empty_bar(buf), 0));
            }
            if (!ok) break;
            if (prm.staged) {
                low_emit_staged<KIND, CPT>(prm, &map_d, smem_base + (uint32_t)(S * Cfg::kStageBytes + (warp - 4) * 4096),
                                           m0 + quarter * 32, n0 + half * CPT, sum, bias_lane, lane);
                continue;
            }
            const int row = m0 + quarter * 32 + lane;
            if (row < prm.m) {
#pragma unroll
                for (int g = 0; g < CPT / 4; g++) {
                    const int col = n0 + half * CPT + g * 4;
                    if (col < prm.n) low_emit4<KIND>(prm, row, col, sum[g * 4], sum[g * 4 + 1], sum[g * 4 + 2], sum[g * 4 + 3], vec_ok);
                }
            }
        }
        if (prm.staged) staged_drain(lane);
    }

    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();     // neither block frees tensor memory or leaves while the partner may still signal it
    if (threadIdx.x == 0 && *abort_flag) atomicOr(prm.error_word, ERR_WAIT_TIMEOUT);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

}  // namespace

cudaError_t gemm_exact(cudaStream_t s, int64_t m, int64_t n, int64_t k, const float *a, int64_t a_ms, int64_t a_ks,
                       const float *b, int64_t b_ks, int64_t b_ns, float *c, int64_t c_ms, int64_t c_ns, const GemmEpilogue &ep) {
    if (m == 0 || n == 0) return cudaSuccess;
    dim3 grid((unsigned)((n + XT - 1) / XT), (unsigned)((m + XT - 1) / XT));
    if (grid.y > 65535) return cudaErrorInvalidValue;
    gemm_exact_kernel<<<grid, 256, 0, s>>>(m, n, k, a, a_ms, a_ks, b, b_ks, b_ns, c, c_ms, c_ns, ep);
    return cudaGetLastError();
}

// Holds SMs the way a collective's blocks do: `blocks` blocks of 1024 threads that each take a whole SM's
// shared memory and sleep until `hold_ns` have passed on the global timer.  No flag, no peer: it ends by itself.
__global__ void __launch_bounds__(1024) occupy_kernel(uint64_t hold_ns) {
    extern __shared__ uint8_t held[];
    const uint64_t start = global_timer();
    while (global_timer() - start < hold_ns) __nanosleep(2000);
    if (hold_ns == ~0ull) held[threadIdx.x] = 0;        // keeps the allocation; never true
}
cudaError_t occupy(cudaStream_t s, int blocks, uint64_t hold_ns) {
    if (blocks < 1) return cudaSuccess;
    const int smem = 200 * 1024;
    cudaError_t e = cudaFuncSetAttribute(occupy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    occupy_kernel<<<blocks, 1024, smem, s>>>(hold_ns);
    return cudaGetLastError();
}

cudaError_t wait_probe(cudaStream_t s, uint64_t limit_ns, int *error_word) {
    // never longer than the GEMM kernels' own limit
    wait_probe_kernel<<<1, 32, 0, s>>>(limit_ns < WAIT_LIMIT_NS ? limit_ns : WAIT_LIMIT_NS, error_word);
    return cudaGetLastError();
}

int64_t padded_k(int64_t k) { return (k + KPAD - 1) / KPAD * KPAD; }
int64_t plane_pitch(int64_t k_padded) { return k_padded % 512 == 0 ? k_padded + 32 : k_padded; }

cudaError_t split_planes(cudaStream_t s, const float *src, int64_t rows, int64_t cols, int64_t rs,
                         float *hi, float *lo, int64_t cp) {
    if (rows == 0) return cudaSuccess;
    int vec_ok = (rs & 3) == 0 && ((uintptr_t)src & 15) == 0;
    int64_t total = rows * (cp >> 2);
    int64_t blocks = (total + 255) / 256;
    split_rows_kernel<<<(unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks), 256, 0, s>>>(src, rows, cols, rs, hi, lo, cp, vec_ok);
    return cudaGetLastError();
}

// Test hook: SYNAPTIK_CUDA_TILE_N=64|128|256 pins the tile width (read once).
static int forced_tile_n() {
    static int value = -1;
    if (value < 0) { const char *e = getenv("SYNAPTIK_CUDA_TILE_N"); value = e ? atoi(e) : 0; }
    return value;
}

// Test hook: SYNAPTIK_CUDA_GROUP_N pins the tile columns per group.
static int forced_group_n() {
    static int value = -1;
    if (value < 0) { const char *e = getenv("SYNAPTIK_CUDA_GROUP_N"); value = e ? atoi(e) : 0; }
    return value;
}

static int forced_chunk_kb() {
    static int value = -1;
    if (value < 0) { const char *e = getenv("SYNAPTIK_CUDA_CHUNK_KB"); value = e ? atoi(e) : 0; }
    return value;
}

struct TensorCoreGemm {
    CUtensorMap p_hi, p_lo, q_hi, q_lo;
    int m, n, k_blocks, bn, grid;
    int promote, chunk_kb, pair;
    int p_mn, q_mn;
    int slices, kb_per_slice; int64_t slice_ld;
    int group_n;
    bool single_wave = false;               // two-SM product whose tiles are at most one per SM pair
    // tensor maps of the staged write-out, encoded when the result arrays change (they rarely do)
    mutable StoreMaps stores;
    mutable const void *stored_for[4] = {nullptr, nullptr, nullptr, nullptr};
    mutable int64_t stored_pitch[2] = {0, 0};
};

// SYNAPTIK_CUDA_STAGED=0 keeps the direct stores of the two-SM FP32 kernel (for comparisons).
static bool staged_enabled() {
    static const bool on = [] { const char *v = getenv("SYNAPTIK_CUDA_STAGED"); return !(v && v[0] == '0'); }();
    return on;
}
// Boxes of 32 rows x 32 floats, 128-byte swizzle, over a [rows, cols] FP32 array.
static bool make_store_map(CUtensorMap *map, const float *base, int64_t rows, int64_t cols, int64_t pitch) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Whether this launch can write out through TMA stores, and its tensor maps if so.
static bool prepare_stores(const TensorCoreGemm *g, const TcParams &prm) {
    if (!staged_enabled() || !g->pair || g->slices > 1 || (prm.n & 3) || (prm.ldd & 3) || ((uintptr_t)prm.d & 15)) return false;
    if ((prm.bias && ((uintptr_t)prm.bias & 15)) || (prm.gate && ((uintptr_t)prm.gate & 15)) || (prm.second && ((uintptr_t)prm.second & 15))) return false;
    if (prm.nhi && ((prm.nld & 3) || ((uintptr_t)prm.nhi & 15) || ((uintptr_t)prm.nlo & 15))) return false;
    const void *now[4] = {prm.d, prm.second, prm.nhi, prm.nlo};
    if (!memcmp(now, g->stored_for, sizeof(now)) && g->stored_pitch[0] == prm.ldd && g->stored_pitch[1] == prm.nld) return true;
    if (!make_store_map(&g->stores.d, prm.d, prm.m, prm.n, prm.ldd)) return false;
    if (prm.second && !make_store_map(&g->stores.second, prm.second, prm.m, prm.n, prm.n)) return false;
    if (prm.nhi && (!make_store_map(&g->stores.hi, prm.nhi, prm.m, prm.nld, prm.nld) || !make_store_map(&g->stores.lo, prm.nlo, prm.m, prm.nld, prm.nld))) return false;
    memcpy(g->stored_for, now, sizeof(now));
    g->stored_pitch[0] = prm.ldd; g->stored_pitch[1] = prm.nld;
    return true;
}

TensorCoreGemm *tc_gemm_prepare(const TcOperand &p, const TcOperand &q, int64_t m, int64_t n, int64_t k,
                                int sm_count, int promote, int *status) {
    const int pair_requested = (promote >> 1) & 1;      // bit 1 of the mode: two-SM tiles
    const int may_slice = (promote >> 2) & 1;           // bit 2: the result has no epilogue, the contraction may be split
    const int fine_units = (promote >> 3) & 1;          // bit 3: a product of one wave or less is cut into at least two slices
    const int chunk_requested = (promote >> 8) & 0xff;  // bits 8-15: k-blocks per tensor-memory partial sum, 0 = default
    promote &= 1;
    *status = OK;
    if (m < 1 || n < 1 || k < 1 || m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) { *status = UNSUPPORTED_SHAPE; return nullptr; }
    TensorCoreGemm *g = new TensorCoreGemm();
    g->m = (int)m; g->n = (int)n; g->k_blocks = (int)((k + BK - 1) / BK);
    g->p_mn = p.mn_major; g->q_mn = q.mn_major;
    g->slices = 1; g->kb_per_slice = g->k_blocks; g->slice_ld = (n + 3) / 4 * 4;
    g->group_n = 1 << 30;
    g->promote = promote;
    // Partial-sum length.  The epilogue warps that add the partials also write the finished tile, and
    // the tensor core can run only two partials ahead of them, so short partials stall it at every
    // tile end unless the tile's main loop is very long (the weight gradients, K = batch).  Measured on
    // the 65536 x 4096 x 4096 layers: partials of 128 contraction steps cost 17 % of the step, 512 nothing.
    g->chunk_kb = (g->k_blocks * BK >= 8192 ? 256 : 512) / BK;
    if (chunk_requested > 0) g->chunk_kb = chunk_requested;
    if (forced_chunk_kb() > 0) g->chunk_kb = forced_chunk_kb();
    // tile width: the widest tile has the best operand reuse, but a persistent grid pays for the last
    // partial wave; take the width with the least (waves x width), narrower tiles handicapped a little
    auto cost = [&](int bn) {
        int64_t t = ((m + BM - 1) / BM) * ((n + bn - 1) / bn);
        int64_t waves = (t + sm_count - 1) / sm_count;
        return (double)waves * bn * (bn == 256 ? 1.0 : (bn == 128 ? 1.05 : 1.15));
    };
    g->bn = 64;
    if (n >= 96 && cost(128) <= cost(g->bn)) g->bn = 128;
    if (n >= 192 && cost(256) <= cost(g->bn)) g->bn = 256;
    if (forced_tile_n() == 64 || forced_tile_n() == 128 || forced_tile_n() == 256) g->bn = forced_tile_n();
    int64_t tiles = ((m + BM - 1) / BM) * ((n + g->bn - 1) / g->bn);
    g->grid = (int)(tiles < sm_count ? tiles : sm_count);
    // two-SM tiles (256 x 256 or 256 x 128) when the shape fills them
    g->pair = pair_requested && m >= 2 * BM && n >= 96 && sm_count >= 2;
    if (g->pair) {
        auto pair_cost = [&](int bn) {
            int64_t t = ((m + 2 * BM - 1) / (2 * BM)) * ((n + bn - 1) / bn);
            int64_t waves = (t + sm_count / 2 - 1) / (sm_count / 2);
            return (double)waves * bn * (bn == 256 ? 1.0 : 1.25);   // 128-wide pair tiles are shared-memory bound again
        };
        g->bn = (n >= 192 && pair_cost(256) <= pair_cost(128)) ? 256 : 128;
        // a short product that fits one wave of 256-wide tiles leaves its whole write-out exposed; in two
        // waves of 128-wide tiles the first write-out hides behind the second main loop
        // (4096 x 1024 x 1024: 57 us against 70)
        if (g->bn == 256 && g->k_blocks <= 64 && ((m + 2 * BM - 1) / (2 * BM)) * ((n + 255) / 256) <= sm_count / 2) g->bn = 128;
        if (forced_tile_n() == 128 || forced_tile_n() == 256) g->bn = forced_tile_n();
        int64_t pair_tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + g->bn - 1) / g->bn);
        int64_t pairs = sm_count / 2;
        g->promote = 1;
        // A persistent grid pays for its last partial wave: 256 tiles on 74 pairs take 4 waves for 3.46
        // waves of work.  Splitting the contraction into slices makes the units shorter and the tail
        // smaller (2 slices: 512 units, 7 half-length waves for 6.92); the slices' partial products go to
        // a workspace and are added in a fixed order by a second kernel.
        if (may_slice) {
            double best = 1e30;
            // A product of at most one wave cannot rebalance when another kernel (an all-reduce) holds some of
            // the SMs: its tiles then take two waves.  Cut into slices it has units to spare (fine_units).
            const int first = (fine_units && pair_tiles <= pairs && g->k_blocks >= 128) ? 2 : 1;
            for (int sl = first; sl <= 4; sl++) {
                const int per = (g->k_blocks + sl - 1) / sl;
                if (sl > first && per < 64) break;              // slices shorter than 2048 steps do not pay for their epilogue
                const int64_t units = pair_tiles * ((g->k_blocks + per - 1) / per);
                const int64_t waves = (units + pairs - 1) / pairs;
                const double cost = (double)waves * per * (1.0 + 0.02 * (sl - 1));
                if (cost < best) { best = cost; g->slices = (g->k_blocks + per - 1) / per; g->kb_per_slice = per; }
            }
        }
        const int64_t units = pair_tiles * g->slices;
        g->single_wave = pair_tiles <= pairs;
        g->grid = (int)(2 * (units < pairs ? units : pairs));
        // tile columns per group: about eight, spread evenly, so that the 74 concurrent tiles form a
        // near-square patch (9 row bands x 8 columns) whatever the contraction length.  Measured on the
        // 65536-row layers against plain row-major order, groups of 4 and of 2: groups of 8 are the
        // fastest or tied everywhere, and 15 % faster on the K = 784 layer.
        // A sliced product (a weight gradient: few tiles, very long contraction) keeps plain row-major
        // order: ncu counted 13.7 GB of DRAM reads per 4096 x 4096 x 65536 product that way and 17.4 GB
        // in groups of 8 (same time), against 16.7 -> 8.5 GB for the unsliced 65536 x 4096 x 4096 products.
        const int tiles_n = (int)((n + g->bn - 1) / g->bn);
        const int groups = (tiles_n + 7) / 8;
        g->group_n = g->slices > 1 ? tiles_n : (tiles_n + groups - 1) / groups;
        if (forced_group_n() > 0) g->group_n = forced_group_n();
    }
    const int q_box = g->pair ? g->bn / 2 : g->bn;
    auto maps = [&](const TcOperand &o, int64_t extent, int box_rows, CUtensorMap *hi, CUtensorMap *lo) {
        if (o.mn_major) return make_plane_map_mn(hi, o.hi, k, padded_k(extent), o.pitch, box_rows)
                               && make_plane_map_mn(lo, o.lo, k, padded_k(extent), o.pitch, box_rows);
        return make_plane_map(hi, o.hi, extent, padded_k(k), o.pitch, box_rows) && make_plane_map(lo, o.lo, extent, padded_k(k), o.pitch, box_rows);
    };
    bool ok = maps(p, m, BM, &g->p_hi, &g->p_lo) && maps(q, n, q_box, &g->q_hi, &g->q_lo);
    if (!ok) { delete g; *status = KERNEL_COMPILATION_FAILED; return nullptr; }
    return g;
}

void tc_gemm_release(TensorCoreGemm *g) { delete g; }
int64_t tc_gemm_workspace_floats(const TensorCoreGemm *g) { return g->slices > 1 ? (int64_t)g->slices * g->m * g->slice_ld : 0; }

template <int BN, bool GENERAL>
static cudaError_t launch_tc(cudaStream_t s, const TensorCoreGemm *g, const TcParams &prm, const SliceParams &slc) {
    using Cfg = TileConfig<BN>;
    cudaError_t e = cudaSuccess;
    if (g->pair) {
        if constexpr (BN >= 128) {
            using Pair = PairConfig<BN>;
            const bool staged = prepare_stores(g, prm);
            auto launch_pair = [&](auto kernel) -> cudaError_t {
                // per-device attributes: set on every launch so each GPU of the process has them
                cudaFuncAttributes attr;
                cudaError_t pe = cudaFuncGetAttributes(&attr, kernel);
                if (pe != cudaSuccess) return pe;
                if (attr.numRegs * PROMOTED_THREADS < 128 * 72 + 256 * 216) return cudaErrorLaunchOutOfResources;
                const int smem_bytes = Pair::kSmemBytes + (staged ? STAGING_BYTES : 0);
                pe = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
                if (pe != cudaSuccess) return pe;
                kernel<<<g->grid, PROMOTED_THREADS, smem_bytes, s>>>(g->p_hi, g->p_lo, g->q_hi, g->q_lo, g->stores, prm, slc);
                return cudaSuccess;
            };
            // a sliced product has no epilogue work, so no activation either
            if (g->slices > 1) e = slc.unit_counter ? launch_pair(gemm_tf32x3_pair_kernel<BN, true, true, false, false>) : launch_pair(gemm_tf32x3_pair_kernel<BN, true, false, false, false>);
            else if (staged) e = slc.unit_counter ? launch_pair(gemm_tf32x3_pair_kernel<BN, false, true, GENERAL, true>) : launch_pair(gemm_tf32x3_pair_kernel<BN, false, false, GENERAL, true>);
            else e = slc.unit_counter ? launch_pair(gemm_tf32x3_pair_kernel<BN, false, true, GENERAL, false>) : launch_pair(gemm_tf32x3_pair_kernel<BN, false, false, GENERAL, false>);
            if (e != cudaSuccess) return e;
        } else return cudaErrorInvalidValue;
    } else if (g->promote) {
        // the kernel redistributes registers between its warpgroups (72 and 216 per thread); that only
        // terminates when the launch allocation covers the sum, so check it instead of trusting it
        cudaFuncAttributes attr;
        e = cudaFuncGetAttributes(&attr, gemm_tf32x3_promoted_kernel<BN, GENERAL>);
        if (e != cudaSuccess) return e;
        if (attr.numRegs * PROMOTED_THREADS < 128 * 72 + 256 * 216) return cudaErrorLaunchOutOfResources;
        e = cudaFuncSetAttribute(gemm_tf32x3_promoted_kernel<BN, GENERAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) return e;
        gemm_tf32x3_promoted_kernel<BN, GENERAL><<<g->grid, PROMOTED_THREADS, Cfg::kSmemBytes, s>>>(g->p_hi, g->p_lo, g->q_hi, g->q_lo, prm);
    } else {
        e = cudaFuncSetAttribute(gemm_tf32x3_kernel<BN, GENERAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) return e;
        gemm_tf32x3_kernel<BN, GENERAL><<<g->grid, GEMM_THREADS, Cfg::kSmemBytes, s>>>(g->p_hi, g->p_lo, g->q_hi, g->q_lo, prm);
    }
    return cudaGetLastError();
}

cudaError_t tc_gemm_launch(cudaStream_t s, const TensorCoreGemm *g, float *d, int64_t ldd, const GemmEpilogue &ep, float *workspace,
                           int *unit_counter, int *error_word) {
    TcParams prm;
    SliceParams slc;
    slc.slices = g->slices; slc.kb_per_slice = g->kb_per_slice; slc.ws = workspace; slc.ld = g->slice_ld;
    slc.group_n = g->group_n;
    slc.unit_counter = g->pair ? unit_counter : nullptr;
    if (g->slices > 1 && (!workspace || ep.bias || ep.gate || ep.second || ep.act || ep.plane_hi)) return cudaErrorInvalidValue;
    prm.nhi = ep.plane_hi; prm.nlo = ep.plane_lo; prm.nld = ep.plane_ld;
    prm.p_mn = g->p_mn; prm.q_mn = g->q_mn;
    prm.d = d; prm.ldd = ldd; prm.m = g->m; prm.n = g->n; prm.k_blocks = g->k_blocks;
    const int tile_m = g->pair ? 2 * BM : BM;
    prm.tiles_m = (g->m + tile_m - 1) / tile_m; prm.tiles_n = (g->n + g->bn - 1) / g->bn;
    prm.chunk_kb = g->chunk_kb;
    prm.bias = ep.bias; prm.gate = ep.gate; prm.second = ep.second; prm.act = ep.act; prm.error_word = error_word;
    const bool general = ep.act != 0 && ep.act != (int)Op::RELU;
    cudaError_t e;
    if (general) e = g->bn == 256 ? launch_tc<256, true>(s, g, prm, slc) : g->bn == 128 ? launch_tc<128, true>(s, g, prm, slc) : launch_tc<64, true>(s, g, prm, slc);
    else e = g->bn == 256 ? launch_tc<256, false>(s, g, prm, slc) : g->bn == 128 ? launch_tc<128, false>(s, g, prm, slc) : launch_tc<64, false>(s, g, prm, slc);
    if (e != cudaSuccess || g->slices <= 1) return e;
    const int64_t total = (int64_t)g->m * (g->slice_ld >> 2);
    const int64_t blocks = (total + 255) / 256;
    slice_combine_kernel<<<(unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks), 256, 0, s>>>(workspace, g->slices, g->m, g->n, g->slice_ld, d, ldd);
    return cudaGetLastError();
}
int tc_gemm_launches(const TensorCoreGemm *g) { return g->slices > 1 ? 2 : 1; }
bool tc_gemm_single_wave(const TensorCoreGemm *g) { return g->pair && g->slices == 1 && g->single_wave; }
bool tc_gemm_staged_shape(const TensorCoreGemm *g) { return staged_enabled() && g->pair && g->slices == 1 && (g->n & 3) == 0; }

// ---- 16-bit storage ------------------------------------------------------------------------------
cudaError_t gemm_exact_low(cudaStream_t s, int kind, int64_t m, int64_t n, int64_t k, const void *a, int64_t a_ms, int64_t a_ks,
                           const void *b, int64_t b_ks, int64_t b_ns, void *c, int64_t c_ms, int64_t c_ns,
                           const void *bias, int act, void *second) {
    if (m == 0 || n == 0) return cudaSuccess;
    dim3 grid((unsigned)((n + XT - 1) / XT), (unsigned)((m + XT - 1) / XT));
    if (grid.y > 65535 || (kind != 1 && kind != 2)) return cudaErrorInvalidValue;
    LowEpilogue ep{(const uint16_t *)bias, act, (uint16_t *)second};
    if (kind == 1) gemm_exact_low_kernel<1><<<grid, 256, 0, s>>>(m, n, k, (const uint16_t *)a, a_ms, a_ks, (const uint16_t *)b, b_ks, b_ns, (uint16_t *)c, c_ms, c_ns, ep);
    else gemm_exact_low_kernel<2><<<grid, 256, 0, s>>>(m, n, k, (const uint16_t *)a, a_ms, a_ks, (const uint16_t *)b, b_ks, b_ns, (uint16_t *)c, c_ms, c_ns, ep);
    return cudaGetLastError();
}

bool low_gemm_supported(int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldw, int64_t ldc) {
    // TMA needs 16-byte row pitches (8 elements); the kernel's tiles need nothing else (edges read as zeros)
    return m >= 1 && n >= 1 && k >= 8 && (k & 7) == 0 && (lda & 7) == 0 && (ldw & 7) == 0 && ldc >= n
           && m < (1ll << 30) && n < (1ll << 30) && k < (1ll << 30);
}

static bool make_low_map(CUtensorMap *map, int kind, const void *base, int64_t rows, int64_t k, int64_t pitch, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {(cuuint32_t)LOW_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// SYNAPTIK_CUDA_LOW_STAGED=0 keeps the direct stores of the 16-bit kernels (for comparisons).
static bool low_staged_enabled() {
    static const bool on = [] { const char *v = getenv("SYNAPTIK_CUDA_LOW_STAGED"); return !(v && v[0] == '0'); }();
    return on;
}
// SYNAPTIK_CUDA_LOW_PAIR=0 keeps 16-bit products on the one-SM kernel (for comparisons).
static bool low_pair_enabled() {
    static const bool on = [] { const char *v = getenv("SYNAPTIK_CUDA_LOW_PAIR"); return !(v && v[0] == '0'); }();
    return on;
}

// Tensor map of the result for the staged write-out: boxes of 32 rows x 64 columns, 128-byte swizzle.
static bool make_low_store_map(CUtensorMap *map, const void *base, int64_t rows, int64_t cols, int64_t pitch) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int KIND>
static cudaError_t launch_low(cudaStream_t s, int grid, const CUtensorMap &p, const CUtensorMap &q, const CUtensorMap &d, const LowParams &prm) {
    using Cfg = LowConfig<BN>;
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, gemm_low_kernel<BN, KIND>);
    if (e != cudaSuccess) return e;
    if (attr.numRegs * PROMOTED_THREADS < 128 * 72 + 256 * 216) return cudaErrorLaunchOutOfResources;
    e = cudaFuncSetAttribute(gemm_low_kernel<BN, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    gemm_low_kernel<BN, KIND><<<grid, PROMOTED_THREADS, Cfg::kSmemBytes, s>>>(p, q, d, prm);
    return cudaGetLastError();
}

template <int KIND>
static cudaError_t launch_low_pair(cudaStream_t s, int grid, const CUtensorMap &p, const CUtensorMap &q, const CUtensorMap &d, const LowParams &prm, int group_n) {
    using Cfg = LowPairConfig;
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, gemm_low_pair_kernel<KIND>);
    if (e != cudaSuccess) return e;
    if (attr.numRegs * PROMOTED_THREADS < 128 * 72 + 256 * 216) return cudaErrorLaunchOutOfResources;
    e = cudaFuncSetAttribute(gemm_low_pair_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    gemm_low_pair_kernel<KIND><<<grid, PROMOTED_THREADS, Cfg::kSmemBytes, s>>>(p, q, d, prm, group_n);
    return cudaGetLastError();
}

cudaError_t low_gemm_launch(cudaStream_t s, int kind, int sm_count, int64_t m, int64_t n, int64_t k, const void *a, int64_t lda,
                            const void *w, int64_t ldw, void *c, int64_t ldc, const void *bias, int act, void *second,
                            int chunk_steps, int *error_word) {
    if ((kind != 1 && kind != 2) || !low_gemm_supported(m, n, k, lda, ldw, ldc)) return cudaErrorInvalidValue;
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return cudaErrorInvalidValue;
    // Kernel and tile width by least (waves x width x cost per column).  A one-SM block loads and reads
    // (128 + BN) x 128 bytes of shared memory per 2 BN clocks of MMA, which narrow tiles cannot sustain; measured
    // clocks per tile column relative to the two-SM kernel on K = 4096 products: 1.2 (BN = 256), 1.8 (128), about
    // 2.5 (64).
    auto cost = [&](int bn) {
        int64_t t = ((m + BM - 1) / BM) * ((n + bn - 1) / bn);
        int64_t waves = (t + sm_count - 1) / sm_count;
        return (double)waves * bn * (bn == 256 ? 1.2 : (bn == 128 ? 1.8 : 2.5));
    };
    int bn = 64;
    if (n >= 96 && cost(128) <= cost(bn)) bn = 128;
    if (n >= 192 && cost(256) <= cost(bn)) bn = 256;
    const int pairs = sm_count / 2;
    const int64_t pair_tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + 255) / 256);
    bool pair = false;
    if (low_pair_enabled() && pairs > 0 && m > BM && n >= 192) {
        const double pair_cost = (double)((pair_tiles + pairs - 1) / pairs) * 256.0;
        if (pair_cost <= cost(bn)) { pair = true; bn = 256; }
    }
    CUtensorMap map_p, map_q;
    if (!make_low_map(&map_p, kind, a, m, k, lda, BM) || !make_low_map(&map_q, kind, w, n, k, ldw, pair ? bn / 2 : bn)) return cudaErrorInvalidValue;
    LowParams prm;
    prm.d = (uint16_t *)c; prm.ldd = ldc; prm.m = (int)m; prm.n = (int)n;
    prm.k_blocks = (int)((k + LOW_BK - 1) / LOW_BK);
    prm.tiles_m = (int)((m + BM - 1) / BM); prm.tiles_n = (int)((n + bn - 1) / bn);
    // A sum kept in tensor memory drifts by about 0.2 * (steps) * 2^-24 of itself (the MMA's accumulation
    // truncates): over 4096 steps that is 5e-5, far below the storage types' own 2^-9 / 2^-12, so a 16-bit
    // result needs no promotion until the contraction is much longer; one partial per 4096 steps keeps the
    // write-out of a tile entirely under the next tile's main loop.
    if (chunk_steps <= 0) chunk_steps = 4096;
    prm.chunk_kb = chunk_steps / LOW_BK < 1 ? 1 : chunk_steps / LOW_BK;
    prm.ep = LowEpilogue{(const uint16_t *)bias, act, (uint16_t *)second};
    prm.error_word = error_word;
    // write-out through shared memory and TMA stores when the result can be described by a tensor map
    // (16-byte pitch and base) and only one tensor is written
    CUtensorMap map_d;
    prm.staged = low_staged_enabled() && bn >= 128 && !second && (ldc & 7) == 0 && ((uintptr_t)c & 15) == 0
                 && make_low_store_map(&map_d, c, m, n, ldc);
    if (!prm.staged) map_d = map_p;         // unused then
    if (pair) {
        prm.tiles_m = (int)((m + 2 * BM - 1) / (2 * BM));
        const int groups = (prm.tiles_n + 7) / 8;
        const int group_n = (prm.tiles_n + groups - 1) / groups;
        const int grid = 2 * (int)(pair_tiles < pairs ? pair_tiles : pairs);
        return kind == 1 ? launch_low_pair<1>(s, grid, map_p, map_q, map_d, prm, group_n) : launch_low_pair<2>(s, grid, map_p, map_q, map_d, prm, group_n);
    }
    const int64_t tiles = (int64_t)prm.tiles_m * prm.tiles_n;
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    if (kind == 1) return bn == 256 ? launch_low<256, 1>(s, grid, map_p, map_q, map_d, prm) : bn == 128 ? launch_low<128, 1>(s, grid, map_p, map_q, map_d, prm) : launch_low<64, 1>(s, grid, map_p, map_q, map_d, prm);
    return bn == 256 ? launch_low<256, 2>(s, grid, map_p, map_q, map_d, prm) : bn == 128 ? launch_low<128, 2>(s, grid, map_p, map_q, map_d, prm) : launch_low<64, 2>(s, grid, map_p, map_q, map_d, prm);
}

}  // namespace kern
}  // namespace syn
