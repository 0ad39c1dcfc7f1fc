// 2-bit / 1-bit matmul for five to sixteen activation rows (sm_100a): the exact int32 block sums of
// matmul_q2 / matmul_q1 (run_q2_gemv, csrc/gemm_q2.cc:300-404; block_sums, src/kernels/lowbit/matmul.rs:373-421)
// formed by warp-level tensor-core instructions, then the reference's ordered fold.
//
// Between the one-wave dp4a kernels (one to four rows, gemv_direct.cu) and the tcgen05 kernel (seventeen rows
// up, lowbit_tc.cu) a call is still a few microseconds of weight streaming, but dp4a would need a
// multiply-add instruction per four weights and row: eight rows of a 4096 x 14336 sign matrix are 117 M dp4a,
// longer than the stream.  mma.m16n8k16 takes the packed unit's lane vector as its A fragment as it lies in
// memory (16 weight columns = M, up to 8 activation rows = N), so the cost per weight no longer grows with the rows.
//
// Exactness.  The int8 tensor path of this part is slow, so the products run in f16 with f32 accumulation and are
// still exact integers: an activation code q (|q| <= 128) is the f16 number q; a weight is the f16 SUBNORMAL whose
// bit pattern is u (1-bit: the sign bit itself, u in {0,1}; 2-bit: codebook value + 128, u in 0..255), i.e. u * 2^-24.
// Every product u q 2^-24 and every partial sum of up to 512 depths (|sum| < 2^24 units) is exact in f32, so
// S = (int)(acc * 2^24) = sum u q, and the block sum is 2 S - sum q (1-bit) or S - 128 sum q (2-bit).  Accumulators are
// drained into integers after every packed unit (128 or 256 depths).  The 1-bit form does not even move its sign bits:
// bit b of a half word is the f16 number 2^(b-24) for b < 12, so a register of the A fragment is the packed word under
// one mask, and act_quant_kernel leaves the codes of the matching depths scaled by the inverse power of two (2^8, 2^0,
// 2^6, 2^-2: still exact f16 numbers), which makes every product u q 2^-16 for one column of a lane and u q 2^-15 for
// the other.
//
// Structure: one CTA of four warps per column group (16 columns) at a time, the warps splitting the depth; small CTAs,
// so that an SM holds a dozen of them and their latencies overlap (a call of this size is latency, not bandwidth).
// A lane copies its own 16 bytes of every unit into its own slot of its warp's shared-memory ring (cp.async; a warp's
// whole share is in flight at once for depths up to 8192), the group's scale rows ride along, and the B fragments are
// 16-byte loads of the activation codes that act_quant_kernel left as f16 in fragment order (64 KB at most, L1
// resident).  The exact block sums meet in shared memory (integer adds: any order), and after a barrier one thread per
// output cell folds its blocks in K order: total = fmaf((float)sum, scale * sa, total), the reference's bits.
#include "epilogue.cuh"
#include "kernels.h"
#include "layout.h"

namespace smeg {
namespace {

constexpr int kMWarps = 4;
constexpr int kMThreads = 32 * kMWarps;
constexpr int kMPF = 8;                                            // units in flight per warp
// ring slots per warp: no more than the units a warp walks per column group (a smaller CTA lets an SM hold one more)
__host__ __device__ inline int ring_units(int upw) { return upw < kMPF ? (upw < 1 ? 1 : upw) : kMPF; }

__device__ __forceinline__ void cpa16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// D (16 weight columns x 8 rows, f32) += A (16 x 16 f16, row-major fragment) * B (16 x 8 f16, column-major fragment)
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// NT = tiles of eight activation rows (1 or 2).  BIGBLK: K-blocks of a whole unit or more.
template <int BITS, int NT, int BIGBLK>
__global__ void __launch_bounds__(kMThreads) lowbit_mma_kernel(const __grid_constant__ LowbitGemvArgs p) {
    constexpr int UD = BITS == 2 ? kQ2UnitDepth : kQ1UnitDepth;
    constexpr int STEPS = UD / 32;
    constexpr int PF = kMPF;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int M = p.m, kq = p.kq, nb = p.nb, ku = p.ku;
    const int pfu = ring_units(p.dupw);
    uint4* ring_w = reinterpret_cast<uint4*>(smem_raw) + (size_t)warp * pfu * 32 + lane;     // + slot * 32
    uint16_t* SCs = reinterpret_cast<uint16_t*>(smem_raw + (size_t)kMWarps * pfu * 512);      // [nb][16] this group's scale rows
    float* SAs = reinterpret_cast<float*>(SCs + (size_t)nb * 16);                             // [M][nb]
    int* QSs = reinterpret_cast<int*>(SAs + (size_t)M * nb);                                  // [M][nb]
    int* sums = QSs + (size_t)M * nb;                                                         // [nb][M][16]
    const int upw = p.dupw;
    const int u_begin = min(warp * upw, ku), u_end = min(u_begin + upw, ku);
    const int mine = u_end - u_begin;
    const uint32_t lutu = p.lut ^ 0x80808080u;                     // codebook value + 128 per code
    const uint16_t* xrow[NT];                                       // this lane's activation row of each tile (row g)
#pragma unroll
    for (int n = 0; n < NT; ++n) xrow[n] = p.qh + (size_t)(8 * n + g) * kq + 8 * t;      // (rows past m are zero rows of qh)
    // steps of a unit that end a K-block (blocks of 32 depths and up but shorter than a unit; units start on block boundaries)
    unsigned end_steps = 0;
    for (int s2 = 0; s2 < STEPS; ++s2)
        if (((32 * (s2 + 1)) & ((1 << p.log2_block) - 1)) == 0) end_steps |= 1u << s2;
    pdl_launch_dependents();
    // a group's scale rows and this warp's first ring-full of units
    auto issue_group = [&](int cg) {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.scales + (size_t)cg * nb * 16);
        for (int ch = tid; ch < nb * 2; ch += kMThreads) cpa16(reinterpret_cast<unsigned char*>(SCs) + ch * 16, src + (size_t)ch * 16);
        const unsigned char* lp = p.codes + ((size_t)cg * ku + u_begin) * kUnitBytes + lane * 16;
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            if (i < mine) cpa16(ring_w + i * 32, lp + (size_t)i * kUnitBytes);
            cpa_commit();
        }
    };
    // the first group's weights leave at once: they do not depend on the kernel ahead in the stream, the activation
    // codes do
    if ((int)blockIdx.x < p.n16) issue_group((int)blockIdx.x);
    for (int idx = tid; idx < nb * M * 16; idx += kMThreads) sums[idx] = 0;
    pdl_wait();
    for (int idx = tid; idx < M * nb; idx += kMThreads) {
        SAs[idx] = p.sa[idx];
        QSs[idx] = p.qsum[idx];
    }
    __syncthreads();

    for (int cg = (int)blockIdx.x; cg < p.n16; cg += (int)gridDim.x) {
        const unsigned char* lp = p.codes + ((size_t)cg * ku + u_begin) * kUnitBytes + lane * 16;
        float acc[NT][4];
        int iacc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) { acc[n][j] = 0.0f; iacc[n][j] = 0; }
        // the accumulators (exact integers scaled by 2^-24) into the integer sums
        auto drain = [&]() {
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // 2-bit: sums scaled by 2^-24; 1-bit: by 2^-16 (columns g: j = 0, 1) and 2^-15 (columns g + 8)
                    iacc[n][j] += __float2int_rn(acc[n][j] * (BITS == 2 ? 16777216.0f : (j < 2 ? 65536.0f : 32768.0f)));
                    acc[n][j] = 0.0f;
                }
        };
        // this warp's share of K-block bl is complete: add it to the block's cells -- weight columns g (j = 0, 1) and
        // g + 8 (j = 2, 3), rows 8 n + 2 t + (j & 1)
        auto flush = [&](int bl) {
            drain();
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = 8 * n + 2 * t + (j & 1), v = iacc[n][j];
                    iacc[n][j] = 0;
                    if (r < M && v != 0) atomicAdd(&sums[((size_t)bl * M + r) * 16 + g + 8 * (j >> 1)], v);
                }
        };
        int slot = 0;
        for (int cu = u_begin; cu < u_end; ++cu) {
            cpa_wait<PF - 1>();                                    // this lane's copy of the unit has landed
            const uint4 wv = ring_w[slot * 32];
            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
            uint4 x[NT][STEPS];
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int s = 0; s < STEPS; ++s) {
                    x[n][s] = __ldg(reinterpret_cast<const uint4*>(xrow[n] + (size_t)cu * UD + 32 * s));
                }
#pragma unroll
            for (int s = 0; s < STEPS; ++s) {
                const int d = cu * UD + 32 * s;                    // the step's 32 depths
                const uint32_t w = words[BITS == 2 ? s : (s >> 1)];
                uint32_t a[2][4];                                  // the A fragments of the step's two instructions
                if (BITS == 2) {
                    const uint32_t e = w & 0x33333333u, o = (w >> 2) & 0x33333333u;
                    const uint32_t glo = prmt(lutu, 0u, e), ghi = prmt(lutu, 0u, e >> 16);      // column g, depths 0-3 / 4-7
                    const uint32_t hlo = prmt(lutu, 0u, o), hhi = prmt(lutu, 0u, o >> 16);      // column g + 8
                    a[0][0] = prmt(glo, 0u, 0x4140u); a[0][1] = prmt(hlo, 0u, 0x4140u);
                    a[0][2] = prmt(glo, 0u, 0x4342u); a[0][3] = prmt(hlo, 0u, 0x4342u);
                    a[1][0] = prmt(ghi, 0u, 0x4140u); a[1][1] = prmt(hhi, 0u, 0x4140u);
                    a[1][2] = prmt(ghi, 0u, 0x4342u); a[1][3] = prmt(hhi, 0u, 0x4342u);
                } else {
                    // A sign bit stays where it lies in its half word: bit b of an f16 is the number 2^(b-24) for
                    // b < 12 (subnormals, then the two smallest exponents), and act_quant_kernel has scaled the codes of
                    // the matching depths by 2^8, 2^0, 2^6, 2^-2, so every product of weight column g is u q 2^-16 and
                    // of column g + 8 (one bit higher) u q 2^-15: one AND per register instead of a shift and an AND.
                    const uint32_t v = w >> (4 * (s & 1));
                    a[0][0] = v & 0x00010001u; a[0][1] = v & 0x00020002u;          // depths (0, 2), codes x 2^8
                    a[0][2] = v & 0x01000100u; a[0][3] = v & 0x02000200u;          // depths (1, 3), codes x 2^0
                    a[1][0] = v & 0x00040004u; a[1][1] = v & 0x00080008u;          // depths (4, 6), codes x 2^6
                    a[1][2] = v & 0x04000400u; a[1][3] = v & 0x08000800u;          // depths (5, 7), codes x 2^-2
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    mma_f16(acc[n], a[0][0], a[0][1], a[0][2], a[0][3], x[n][s].x, x[n][s].y);
                    mma_f16(acc[n], a[1][0], a[1][1], a[1][2], a[1][3], x[n][s].z, x[n][s].w);
                }
                // end of a K-block (blocks of 32 and up: the whole step lies in one block), or of this warp's share
                if (!BIGBLK && ((end_steps >> s) & 1u)) flush(d >> p.log2_block);
            }
            if (BIGBLK) {
                if ((((cu + 1) * UD) & ((1 << p.log2_block) - 1)) == 0 || cu == u_end - 1) flush((cu * UD) >> p.log2_block);
                else drain();
            }
            if (cu - u_begin + PF < mine) cpa16(ring_w + slot * 32, lp + (size_t)(cu - u_begin + PF) * kUnitBytes);
            cpa_commit();
            slot = slot + 1 == PF ? 0 : slot + 1;
        }
        cpa_wait<0>();                                             // the scale rows (first group of copies) as well
        __syncthreads();
        // ---- ordered fold of the group's cells, epilogue, store; the cells are cleared for the next group ----
        for (int cell = tid; cell < M * 16; cell += kMThreads) {
            const int col16 = cell & 15, r = cell >> 4;
            const int col = cg * 16 + col16;
            const uint16_t* sc = SCs + scale_slot(col16);
            int* cs = sums + (size_t)r * 16 + col16;
            float tot = 0.0f;
#pragma unroll 4
            for (int bl = 0; bl < p.nb_real; ++bl) {
                int sum = cs[(size_t)bl * M * 16];
                cs[(size_t)bl * M * 16] = 0;
                sum = BITS == 1 ? 2 * sum - QSs[r * nb + bl] : sum - 128 * QSs[r * nb + bl];
                if (p.sums_out && col < p.n) p.sums_out[((size_t)r * p.n + col) * p.nb_real + bl] = sum;
                const float scale = __half2float(__ushort_as_half(sc[(size_t)bl * 16]));
                tot = fmaf((float)sum, __fmul_rn(scale, SAs[r * nb + bl]), tot);
            }
            if (col < p.n) p.c[(size_t)r * p.n + col] = ep_store_value<0>(p.ep, tot, (size_t)r, (size_t)col);
        }
        __syncthreads();                                           // the scale rows and cells are free again
        if (cg + (int)gridDim.x < p.n16) issue_group(cg + (int)gridDim.x);
    }
}

size_t mma_smem(const LowbitGemvArgs& a) {
    return (size_t)kMWarps * ring_units((a.ku + kMWarps - 1) / kMWarps) * 512 + (size_t)a.nb * 32 + (size_t)2 * a.m * a.nb * 4 + (size_t)a.nb * a.m * 16 * 4;
}

}  // namespace

bool lowbit_mma_supported(const LowbitGemvArgs& a, int sm_count) {
    (void)sm_count;
    if (a.m < 1 || a.m > 16 || a.ku < 1 || a.k < 1 || a.log2_block < 5) return false;
    return a.qh && a.sa && a.qsum && mma_smem(a) <= 100 * 1024;
}

cudaError_t lowbit_mma_launch(LowbitGemvArgs a, int bits, int sm_count, cudaStream_t stream) {
    // one column group per CTA where the machine holds that many CTAs of this kernel at once
    const size_t smem = mma_smem(a);
    // (a CTA per group up to a few waves: a grid cut to exactly one wave leaves its last groups to run alone)
    int per_sm = (int)((size_t)220 * 1024 / (smem + 1024));
    if (per_sm > 16) per_sm = 16;
    if (per_sm < 1) per_sm = 1;
    const int grid_x = a.n16 < 4 * per_sm * sm_count ? a.n16 : 4 * per_sm * sm_count;
    a.dupw = (a.ku + kMWarps - 1) / kMWarps;
    const int ud = bits == 2 ? kQ2UnitDepth : kQ1UnitDepth;
    const int big = (1 << a.log2_block) >= ud ? 1 : 0;
    const int nt = a.m > 8 ? 2 : 1;
    const dim3 grid(grid_x);
    cudaError_t e;
#define SMEG_LM(BB, NN, GG)                                                                                        \
    if (bits == BB && nt == NN && big == GG) {                                                                     \
        e = cudaFuncSetAttribute(lowbit_mma_kernel<BB, NN, GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
        if (e != cudaSuccess) return e;                                                                            \
        return launch_pdl(lowbit_mma_kernel<BB, NN, GG>, grid, dim3(kMThreads), smem, stream, a);                  \
    }
    SMEG_LM(1, 1, 0) SMEG_LM(1, 1, 1) SMEG_LM(1, 2, 0) SMEG_LM(1, 2, 1)
    SMEG_LM(2, 1, 0) SMEG_LM(2, 1, 1) SMEG_LM(2, 2, 0) SMEG_LM(2, 2, 1)
#undef SMEG_LM
    return cudaErrorInvalidValue;
}

}  // namespace smeg
