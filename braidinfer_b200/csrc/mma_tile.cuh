// A bfloat16 tile product on the tensor cores (mma.sync m16n8k16, float32 accumulators) for kernels whose
// tiles are found on the device: rows gathered through an index, one matrix per expert or per head.
//
//   C[BM x BN] = A[BM x K] * B[BN x K]^T      A: a pointer per row (null: a row of zeros), k contiguous
//                                             B: rows of a [*, K] matrix, k contiguous ([out, in] weights)
// Both operands are k-major, so fragments come from shared memory with plain ldmatrix.  k runs in blocks of
// 32 through three shared-memory stages filled by cp.async, two blocks ahead of the one being multiplied and
// one barrier a block (16 bytes a copy: K and every row start must be multiples of 8 elements; past K a copy
// is filled with zeros).  NB = 2 multiplies the same A tile with two
// B matrices at once (gate and up of a SwiGLU).  128 threads: WM x WN warps, each a (BM/WM) x (BN/WN) part.
#pragma once
#include "common.cuh"

#define MT_BK 32
#define MT_STAGES 3
#define MT_LDS (MT_BK + 8)      // 80 bytes a row: eight consecutive rows fall into eight different 16-byte columns

__device__ __forceinline__ void mt_cp_async16(void* smem, const void* gmem, int src_bytes) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void mt_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void mt_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mt_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mt_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mt_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int BM, int BN, int WM, int WN, int NB>
struct MmaTile {
    static constexpr int MI = BM / WM / 16;       // m16 tiles a warp
    static constexpr int NI = BN / WN / 8;        // n8 tiles a warp (even)
    static constexpr int A_ELEMS = MT_STAGES * BM * MT_LDS;
    static constexpr int B_ELEMS = MT_STAGES * BN * MT_LDS;
    static constexpr int SMEM_BYTES = (A_ELEMS + NB * B_ELEMS) * 2;
    static_assert(WM * WN == 4 && MI >= 1 && NI >= 2 && NI % 2 == 0, "four warps; at least 16 x 16 a warp");

    // acc[b][mi][ni][4]: element (row g + 8*(e/2), column 2*(lane%4) + e%2) of the warp's tile (mi, ni), g = lane / 4
    // a_rows: for every row chunk this thread copies, the row's start (or null); b_rows likewise for each B.
    // Chunks: thread t copies A chunks t, t + 128, ...: chunk c is row c / 4, 16-byte column c % 4.
    static __device__ __forceinline__ void run(float (&acc)[NB][MI][NI][4], __nv_bfloat16* smem,
                                               const __nv_bfloat16* const* a_rows,      // [BM * 4 / 128] a thread
                                               const __nv_bfloat16* const (*b_rows)[BN * 4 / 128],   // [NB][...]
                                               int K, const void* safe) {     // safe: any global address (never read)
        constexpr int ACH = BM * 4 / 128, BCH = BN * 4 / 128;
        __nv_bfloat16* As = smem;
        __nv_bfloat16* Bs = smem + A_ELEMS;
        const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
        const int wm0 = (warp / WN) * (BM / WM), wn0 = (warp % WN) * (BN / WN);
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                for (int ni = 0; ni < NI; ++ni)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[b][mi][ni][e] = 0.f;
        const int KT = (K + MT_BK - 1) / MT_BK;
        auto load = [&](int kt, int stage) {
            const int k0 = kt * MT_BK;
            if (BM * 4 >= 128) {
#pragma unroll
                for (int i = 0; i < (ACH > 0 ? ACH : 1); ++i) {
                    const int c = tid + i * 128, r = c >> 2, kc = (c & 3) * 8;
                    const __nv_bfloat16* src = a_rows[i];
                    const bool ok = src != nullptr && k0 + kc < K;
                    mt_cp_async16(As + (stage * BM + r) * MT_LDS + kc, ok ? src + k0 + kc : (const __nv_bfloat16*)safe, ok ? 16 : 0);
                }
            } else if (tid < BM * 4) {
                const int r = tid >> 2, kc = (tid & 3) * 8;
                const __nv_bfloat16* src = a_rows[0];
                const bool ok = src != nullptr && k0 + kc < K;
                mt_cp_async16(As + (stage * BM + r) * MT_LDS + kc, ok ? src + k0 + kc : (const __nv_bfloat16*)safe, ok ? 16 : 0);
            }
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int i = 0; i < BCH; ++i) {
                    const int c = tid + i * 128, r = c >> 2, kc = (c & 3) * 8;
                    const __nv_bfloat16* src = b_rows[b][i];
                    const bool ok = src != nullptr && k0 + kc < K;
                    mt_cp_async16(Bs + b * B_ELEMS + (stage * BN + r) * MT_LDS + kc, ok ? src + k0 + kc : (const __nv_bfloat16*)safe, ok ? 16 : 0);
                }
            mt_commit();
        };
        // a group is committed for every block slot, empty where k has ended, so that the wait counts stay uniform
#pragma unroll
        for (int p = 0; p < MT_STAGES - 1; ++p) {
            if (p < KT) load(p, p);
            else mt_commit();
        }
        for (int kt = 0; kt < KT; ++kt) {
            const int stage = kt % MT_STAGES;
            mt_wait<MT_STAGES - 2>();          // block kt has arrived (this thread's copies)
            __syncthreads();                   // ... everybody's; and everybody is done with block kt - 1,
            if (kt + MT_STAGES - 1 < KT) load(kt + MT_STAGES - 1, (kt + MT_STAGES - 1) % MT_STAGES);   // whose stage is filled next
            else mt_commit();
#pragma unroll
            for (int ks = 0; ks < MT_BK / 16; ++ks) {
                unsigned af[MI][4];
#pragma unroll
                for (int mi = 0; mi < MI; ++mi)
                    mt_ldmatrix_x4(af[mi], As + (stage * BM + wm0 + mi * 16 + (lane & 15)) * MT_LDS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int np = 0; np < NI / 2; ++np) {
                        unsigned bf[4];
                        mt_ldmatrix_x4(bf, Bs + b * B_ELEMS + (stage * BN + wn0 + np * 16 + (lane & 7) + (lane >> 4) * 8) * MT_LDS +
                                               ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
                        for (int mi = 0; mi < MI; ++mi) {
                            mt_mma(acc[b][mi][2 * np], af[mi], bf[0], bf[1]);
                            mt_mma(acc[b][mi][2 * np + 1], af[mi], bf[2], bf[3]);
                        }
                    }
            }
        }
        mt_wait<0>();
    }
};
