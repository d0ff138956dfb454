// bfloat16 attention over the latent cache on the tensor cores (mma.sync m16n8k16, float32 scores, softmax and
// accumulators), compiled for one latent size: -DBRAID_LAT_RANK (kv_rank) and -DBRAID_LAT_ROT (rot_dim), both
// multiples of 16.  A cached row [c ; kr] (D = rank + rot numbers) is the key of every head; its first `rank`
// numbers are the value (see latent.cu for why).  All heads of a token share the keys, so the rows of a tile are
// (token, head) pairs: a decoded token alone fills the tensor cores' M with its heads.
//
// One CTA: 64 (token, head) pairs of one sequence (4 warps x 16), up to 256 value columns (a larger rank is cut
// into column parts, grid.z, each recomputing the scores), one slice of the context (grid.z too).  Keys arrive
// 32 at a time (half a page) through two cp.async stages; scores S = Q K^T with Q fragments read from shared
// memory, the online softmax in registers, P reused as the A operand of O += P V with V fragments taken from
// the same key tile by transposing loads.  With slices, unnormalised O and (max, sum) go to a workspace and a
// second kernel merges them.  Key j is visible to position p iff j <= p and (no window or p - j < window).
#include "common.cuh"
#include "mma_tile.cuh"
#include "page.h"

#ifndef BRAID_LAT_RANK
#error "compile with -DBRAID_LAT_RANK=<kv_rank> -DBRAID_LAT_ROT=<rot_dim>"
#endif

namespace {
constexpr int R = BRAID_LAT_RANK, RT = BRAID_LAT_ROT, D = R + RT;
constexpr int VC = R <= 256 ? R : 256;            // value columns a CTA
constexpr int VPARTS = R / VC;
constexpr int BM = 64, BN = 32, LDK = D + 8;      // (D + 8) * 2 bytes a row: conflict-free for ldmatrix when D % 16 == 0
constexpr int SMEM_BYTES = (BM + 2 * BN) * LDK * 2;
static_assert(R % 16 == 0 && RT % 16 == 0 && R > 0, "kv_rank and rot_dim must be multiples of 16");
static_assert(R % VC == 0, "a kv_rank above 256 must be a multiple of 256");
static_assert(BRAID_PAGE_SIZE % BN == 0, "a key tile lies within one page");
}

struct LatAttnArgs {
    const __nv_bfloat16* q;        // [rows, heads, D] contiguous
    __nv_bfloat16* out;            // [rows, heads, R] contiguous
    float* partial;                // slices: [n_splits][rows * heads][R + 4], else null
    const __nv_bfloat16* cache;    // [pages][page_size][D]
    const int* page_table;         // [n_seqs, table_cols]
    const int* q_start;
    const int* q_len;
    const int* kv_before;
    int heads, table_cols, num_pages, window, n_splits, total_pairs;
    float scale_log2;              // scale * log2(e)
    int* error_flag;
};

__global__ void __launch_bounds__(128)
latent_attn_mma_kernel(LatAttnArgs a) {
    extern __shared__ __align__(16) unsigned char lat_smem[];
    __nv_bfloat16* Qs = (__nv_bfloat16*)lat_smem;
    __nv_bfloat16* Ks = Qs + BM * LDK;
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y;
    const int split = blockIdx.z / VPARTS, vc0 = (blockIdx.z % VPARTS) * VC;
    const int n_q = a.q_len[seq];
    const int pairs = n_q * a.heads;
    const int pair0 = blockIdx.x * BM;
    if (pair0 >= pairs) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int before = a.kv_before[seq];
    const long long base_pair = (long long)a.q_start[seq] * a.heads + pair0;     // index of the tile's first pair in the step
    const int n_here = min(BM, pairs - pair0);

    // keys this tile can see, and this CTA's slice of them (in tiles of BN keys)
    const int t_first = pair0 / a.heads, t_last = (pair0 + n_here - 1) / a.heads;
    const int hi = before + t_last;
    int lo = 0;
    if (a.window > 0 && before + t_first - a.window + 1 > 0) lo = before + t_first - a.window + 1;
    const int tile_lo = lo / BN, tile_hi = hi / BN;                                // inclusive
    const int n_tiles = tile_hi - tile_lo + 1;
    const int per = (n_tiles + a.n_splits - 1) / a.n_splits;
    const int my_lo = tile_lo + split * per;
    const int my_hi = min(tile_hi, my_lo + per - 1);

    // Q tile: n_here consecutive rows of D numbers
    {
        const __nv_bfloat16* src = a.q + base_pair * D;
        constexpr int CH = D / 8;
        for (int c = tid; c < BM * CH; c += 128) {
            const int r = c / CH, kc = (c - r * CH) * 8;
            const bool ok = r < n_here;
            mt_cp_async16(Qs + r * LDK + kc, ok ? src + (size_t)r * D + kc : a.q, ok ? 16 : 0);
        }
    }
    const int* table = a.page_table + (size_t)seq * a.table_cols;
    auto load_keys = [&](int tile, int stage) {
        const int j0 = tile * BN;
        const int block = j0 / BRAID_PAGE_SIZE, off = j0 - block * BRAID_PAGE_SIZE;
        int page = (block < a.table_cols) ? table[block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (tid == 0) atomicExch(a.error_flag, 1);
            page = 0;
        }
        const __nv_bfloat16* src = a.cache + ((size_t)page * BRAID_PAGE_SIZE + off) * D;
        constexpr int CH = D / 8;
        __nv_bfloat16* dst = Ks + stage * BN * LDK;
        for (int c = tid; c < BN * CH; c += 128) {
            const int r = c / CH, kc = (c - r * CH) * 8;
            mt_cp_async16(dst + r * LDK + kc, src + (size_t)r * D + kc, 16);
        }
    };
    if (my_lo <= my_hi) load_keys(my_lo, 0);
    mt_commit();

    // the two rows of this thread: g and g + 8 of the warp's sixteen
    const int g = lane >> 2, qd = lane & 3;
    int pos_row[2];
    bool live_row[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int idx = warp * 16 + g + h2 * 8;
        live_row[h2] = idx < n_here;
        pos_row[h2] = before + (pair0 + idx) / a.heads;
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[VC / 8][4];
#pragma unroll
    for (int i = 0; i < VC / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;

    for (int tile = my_lo; tile <= my_hi; ++tile) {
        const int stage = (tile - my_lo) & 1;
        if (tile + 1 <= my_hi) {
            load_keys(tile + 1, stage ^ 1);
            mt_commit();
            mt_wait<1>();
        } else {
            mt_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* Kt = Ks + stage * BN * LDK;
        float sacc[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
#pragma unroll 4
        for (int kd = 0; kd < D / 16; ++kd) {
            unsigned af[4];
            mt_ldmatrix_x4(af, Qs + (warp * 16 + (lane & 15)) * LDK + kd * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                unsigned bf[4];
                mt_ldmatrix_x4(bf, Kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + kd * 16 + ((lane >> 3) & 1) * 8);
                mt_mma(sacc[2 * np], af, bf[0], bf[1]);
                mt_mma(sacc[2 * np + 1], af, bf[2], bf[3]);
            }
        }
        // mask, scale, online softmax
        const int j0 = tile * BN;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int ni = 0; ni < BN / 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h2 = e >> 1;
                const int j = j0 + ni * 8 + 2 * qd + (e & 1);
                const bool vis = live_row[h2] && j <= pos_row[h2] && (a.window <= 0 || pos_row[h2] - j < a.window);
                const float s = vis ? sacc[ni][e] * a.scale_log2 : -INFINITY;
                sacc[ni][e] = s;
                mx[h2] = fmaxf(mx[h2], s);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
            const float m_new = fmaxf(m_run[h2], mx[h2]);
            m_use[h2] = (m_new == -INFINITY) ? 0.f : m_new;
            corr[h2] = exp2f(m_run[h2] - m_use[h2]);             // m_run = -inf: 0
            m_run[h2] = m_new;
            l_run[h2] *= corr[h2];
        }
        unsigned pf[BN / 16][4];
#pragma unroll
        for (int ni = 0; ni < BN / 8; ++ni) {
            const float p0 = exp2f(sacc[ni][0] - m_use[0]), p1 = exp2f(sacc[ni][1] - m_use[0]);
            const float p2 = exp2f(sacc[ni][2] - m_use[1]), p3 = exp2f(sacc[ni][3] - m_use[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            __nv_bfloat162 lo2 = __floats2bfloat162_rn(p0, p1), hi2 = __floats2bfloat162_rn(p2, p3);
            pf[ni >> 1][(ni & 1) * 2] = *reinterpret_cast<unsigned*>(&lo2);
            pf[ni >> 1][(ni & 1) * 2 + 1] = *reinterpret_cast<unsigned*>(&hi2);
        }
#pragma unroll
        for (int i = 0; i < VC / 8; ++i) {
            oacc[i][0] *= corr[0]; oacc[i][1] *= corr[0];
            oacc[i][2] *= corr[1]; oacc[i][3] *= corr[1];
        }
        // O += P V: V[key][col] is the key tile's columns vc0 .. vc0 + VC
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int np = 0; np < VC / 16; ++np) {
                unsigned bf[4];
                mt_ldmatrix_x4_trans(bf, Kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + vc0 + np * 16 + (lane >> 4) * 8);
                mt_mma(oacc[2 * np], pf[kk], bf[0], bf[1]);
                mt_mma(oacc[2 * np + 1], pf[kk], bf[2], bf[3]);
            }
        }
        __syncthreads();
    }
    if (my_lo > my_hi) mt_wait<0>();
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        if (!live_row[h2]) continue;
        const long long pair = base_pair + warp * 16 + g + h2 * 8;
        if (a.partial == nullptr) {
            const float inv = 1.f / l_run[h2];
            __nv_bfloat16* o = a.out + pair * R + vc0;
#pragma unroll
            for (int i = 0; i < VC / 8; ++i)
                *reinterpret_cast<__nv_bfloat162*>(o + i * 8 + 2 * qd) = __floats2bfloat162_rn(oacc[i][h2 * 2] * inv, oacc[i][h2 * 2 + 1] * inv);
        } else {
            float* o = a.partial + ((size_t)split * a.total_pairs + pair) * (R + 4);
#pragma unroll
            for (int i = 0; i < VC / 8; ++i)
                *reinterpret_cast<float2*>(o + vc0 + i * 8 + 2 * qd) = make_float2(oacc[i][h2 * 2], oacc[i][h2 * 2 + 1]);
            if (qd == 0 && vc0 == 0) {
                o[R] = m_run[h2];
                o[R + 1] = l_run[h2];
            }
        }
    }
}

// ------------------------------------------------------------------ steps of few (token, head) pairs
// A decoded token of a model with few heads fills one m16 tile at most, so the four warps of a CTA share the same
// sixteen rows instead of taking sixteen each: they split the scores' sum over the D numbers of a key (warp w takes
// every fourth block of 16; partial scores meet in shared memory), every warp then holds all scores, runs the same
// softmax, and accumulates its own quarter of the value columns.  No product is computed twice, and a rank above 256
// needs no column parts.  Built where kv_rank is a multiple of 64.
namespace {
constexpr bool FEW_OK = (R % 64 == 0);
constexpr int VQ = FEW_OK ? R / 4 : 16;
constexpr int FEW_ROWS = 16;
constexpr int SP_LD = BN + 1;
constexpr int SMEM_FEW = (FEW_ROWS + 2 * BN) * LDK * 2 + 2 * 4 * FEW_ROWS * SP_LD * 4;
}

__global__ void __launch_bounds__(128)
latent_attn_few_kernel(LatAttnArgs a) {
    extern __shared__ __align__(16) unsigned char lat_smem[];
    __nv_bfloat16* Qs = (__nv_bfloat16*)lat_smem;
    __nv_bfloat16* Ks = Qs + FEW_ROWS * LDK;
    float* Sp = (float*)(Ks + 2 * BN * LDK);             // [2][4 warps][16][SP_LD]
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y, split = blockIdx.z;
    const int pairs = a.q_len[seq] * a.heads;
    const int pair0 = blockIdx.x * FEW_ROWS;
    if (pair0 >= pairs) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int before = a.kv_before[seq];
    const long long base_pair = (long long)a.q_start[seq] * a.heads + pair0;
    const int n_here = min(FEW_ROWS, pairs - pair0);
    const int t_first = pair0 / a.heads, t_last = (pair0 + n_here - 1) / a.heads;
    const int hi = before + t_last;
    int lo = 0;
    if (a.window > 0 && before + t_first - a.window + 1 > 0) lo = before + t_first - a.window + 1;
    const int tile_lo = lo / BN, tile_hi = hi / BN;
    const int per = (tile_hi - tile_lo + 1 + a.n_splits - 1) / a.n_splits;
    const int my_lo = tile_lo + split * per;
    const int my_hi = min(tile_hi, my_lo + per - 1);
    constexpr int CH = D / 8;
    {
        const __nv_bfloat16* src = a.q + base_pair * D;
        for (int c = tid; c < FEW_ROWS * CH; c += 128) {
            const int r = c / CH, kc = (c - r * CH) * 8;
            const bool ok = r < n_here;
            mt_cp_async16(Qs + r * LDK + kc, ok ? src + (size_t)r * D + kc : a.q, ok ? 16 : 0);
        }
    }
    const int* table = a.page_table + (size_t)seq * a.table_cols;
    auto load_keys = [&](int tile, int stage) {
        const int j0 = tile * BN;
        const int block = j0 / BRAID_PAGE_SIZE, off = j0 - block * BRAID_PAGE_SIZE;
        int page = (block < a.table_cols) ? table[block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (tid == 0) atomicExch(a.error_flag, 1);
            page = 0;
        }
        const __nv_bfloat16* src = a.cache + ((size_t)page * BRAID_PAGE_SIZE + off) * D;
        __nv_bfloat16* dst = Ks + stage * BN * LDK;
        for (int c = tid; c < BN * CH; c += 128) {
            const int r = c / CH, kc = (c - r * CH) * 8;
            mt_cp_async16(dst + r * LDK + kc, src + (size_t)r * D + kc, 16);
        }
    };
    if (my_lo <= my_hi) load_keys(my_lo, 0);
    mt_commit();
    const int g = lane >> 2, qd = lane & 3;
    int pos_row[2];
    bool live_row[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int idx = g + h2 * 8;
        live_row[h2] = idx < n_here;
        pos_row[h2] = before + (pair0 + idx) / a.heads;
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[VQ / 8][4];
#pragma unroll
    for (int i = 0; i < VQ / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
    for (int tile = my_lo; tile <= my_hi; ++tile) {
        const int it = tile - my_lo, stage = it & 1;
        if (tile + 1 <= my_hi) {
            load_keys(tile + 1, stage ^ 1);
            mt_commit();
            mt_wait<1>();
        } else {
            mt_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* Kt = Ks + stage * BN * LDK;
        float sacc[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
        for (int kd = warp; kd < D / 16; kd += 4) {
            unsigned af[4];
            mt_ldmatrix_x4(af, Qs + (lane & 15) * LDK + kd * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                unsigned bf[4];
                mt_ldmatrix_x4(bf, Kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + kd * 16 + ((lane >> 3) & 1) * 8);
                mt_mma(sacc[2 * np], af, bf[0], bf[1]);
                mt_mma(sacc[2 * np + 1], af, bf[2], bf[3]);
            }
        }
        float* mine = Sp + ((it & 1) * 4 + warp) * FEW_ROWS * SP_LD;
#pragma unroll
        for (int ni = 0; ni < BN / 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) mine[(g + (e >> 1) * 8) * SP_LD + ni * 8 + 2 * qd + (e & 1)] = sacc[ni][e];
        __syncthreads();
        const float* all = Sp + (it & 1) * 4 * FEW_ROWS * SP_LD;
        const int j0 = tile * BN;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int ni = 0; ni < BN / 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h2 = e >> 1;
                const int o = (g + h2 * 8) * SP_LD + ni * 8 + 2 * qd + (e & 1);
                const float dot = (all[o] + all[FEW_ROWS * SP_LD + o]) + (all[2 * FEW_ROWS * SP_LD + o] + all[3 * FEW_ROWS * SP_LD + o]);
                const int j = j0 + ni * 8 + 2 * qd + (e & 1);
                const bool vis = live_row[h2] && j <= pos_row[h2] && (a.window <= 0 || pos_row[h2] - j < a.window);
                const float s = vis ? dot * a.scale_log2 : -INFINITY;
                sacc[ni][e] = s;
                mx[h2] = fmaxf(mx[h2], s);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
            mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
            const float m_new = fmaxf(m_run[h2], mx[h2]);
            m_use[h2] = (m_new == -INFINITY) ? 0.f : m_new;
            corr[h2] = exp2f(m_run[h2] - m_use[h2]);
            m_run[h2] = m_new;
            l_run[h2] *= corr[h2];
        }
        unsigned pf[BN / 16][4];
#pragma unroll
        for (int ni = 0; ni < BN / 8; ++ni) {
            const float p0 = exp2f(sacc[ni][0] - m_use[0]), p1 = exp2f(sacc[ni][1] - m_use[0]);
            const float p2 = exp2f(sacc[ni][2] - m_use[1]), p3 = exp2f(sacc[ni][3] - m_use[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            __nv_bfloat162 lo2 = __floats2bfloat162_rn(p0, p1), hi2 = __floats2bfloat162_rn(p2, p3);
            pf[ni >> 1][(ni & 1) * 2] = *reinterpret_cast<unsigned*>(&lo2);
            pf[ni >> 1][(ni & 1) * 2 + 1] = *reinterpret_cast<unsigned*>(&hi2);
        }
#pragma unroll
        for (int i = 0; i < VQ / 8; ++i) {
            oacc[i][0] *= corr[0]; oacc[i][1] *= corr[0];
            oacc[i][2] *= corr[1]; oacc[i][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
#pragma unroll
            for (int np = 0; np < VQ / 16; ++np) {
                unsigned bf[4];
                mt_ldmatrix_x4_trans(bf, Kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + warp * VQ + np * 16 + (lane >> 4) * 8);
                mt_mma(oacc[2 * np], pf[kk], bf[0], bf[1]);
                mt_mma(oacc[2 * np + 1], pf[kk], bf[2], bf[3]);
            }
        __syncthreads();
    }
    if (my_lo > my_hi) mt_wait<0>();
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        if (!live_row[h2]) continue;
        const long long pair = base_pair + g + h2 * 8;
        if (a.partial == nullptr) {
            const float inv = 1.f / l_run[h2];
            __nv_bfloat16* o = a.out + pair * R + warp * VQ;
#pragma unroll
            for (int i = 0; i < VQ / 8; ++i)
                *reinterpret_cast<__nv_bfloat162*>(o + i * 8 + 2 * qd) = __floats2bfloat162_rn(oacc[i][h2 * 2] * inv, oacc[i][h2 * 2 + 1] * inv);
        } else {
            float* o = a.partial + ((size_t)split * a.total_pairs + pair) * (R + 4);
#pragma unroll
            for (int i = 0; i < VQ / 8; ++i)
                *reinterpret_cast<float2*>(o + warp * VQ + i * 8 + 2 * qd) = make_float2(oacc[i][h2 * 2], oacc[i][h2 * 2 + 1]);
            if (qd == 0 && warp == 0) {
                o[R] = m_run[h2];
                o[R + 1] = l_run[h2];
            }
        }
    }
}

// Merge of the context's slices: out = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s, M = max_s m_s.  One CTA a
// (token, head) pair: the slices' (max, sum) pairs are fetched once into shared memory, then every thread adds up
// four columns over the slices with all its loads in flight at once (up to 64 slices).
#define LAT_MERGE_MAX_SPLITS 64
__global__ void __launch_bounds__(128)
latent_attn_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, const int* __restrict__ token_seq,
                         int heads, int total_pairs, int n_splits) {
    pdl_trigger();
    pdl_wait();
    __shared__ float wgt[LAT_MERGE_MAX_SPLITS];
    __shared__ float inv_s;
    const int pair = blockIdx.x;
    if (token_seq[pair / heads] < 0) return;             // a padding row: nothing was computed for it
    const size_t stride = (size_t)total_pairs * (R + 4);
    const float* base = partial + (size_t)pair * (R + 4);
    if (threadIdx.x < 32) {
        float m[2], l[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int s_ = threadIdx.x + 32 * i;
            m[i] = s_ < n_splits ? base[s_ * stride + R] : -INFINITY;
            l[i] = s_ < n_splits ? base[s_ * stride + R + 1] : 0.f;
        }
        const float M = warp_max(fmaxf(m[0], m[1]));
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float w = (m[i] == -INFINITY) ? 0.f : exp2f(m[i] - M);
            if (threadIdx.x + 32 * i < LAT_MERGE_MAX_SPLITS) wgt[threadIdx.x + 32 * i] = w;
            d += w * l[i];
        }
        d = warp_sum(d);
        if (threadIdx.x == 0) inv_s = d > 0.f ? 1.f / d : 0.f;
    }
    __syncthreads();
    const float inv = inv_s;
    for (int c = threadIdx.x * 4; c < R; c += 128 * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int s_ = 0; s_ < n_splits; ++s_) {
            const float4 v = *reinterpret_cast<const float4*>(base + s_ * stride + c);
            const float w = wgt[s_];
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        __nv_bfloat162 a = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), b = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
        uint2 pk;
        pk.x = *reinterpret_cast<unsigned*>(&a);
        pk.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(out + (size_t)pair * R + c) = pk;
    }
}

extern "C" int braid_latent_attn_rank(void) { return R; }
extern "C" int braid_latent_attn_rot(void) { return RT; }
extern "C" int braid_latent_attn_vparts(void) { return VPARTS; }

// Rows of a CTA's tile for a step whose sequences bring up to max_q_len tokens: 16 (the kernel for few pairs) or 64.
extern "C" int braid_latent_attn_tile_rows(int max_q_len, int heads) {
    return (FEW_OK && (long long)max_q_len * heads <= 32) ? FEW_ROWS : BM;
}

extern "C" long long braid_latent_attn_partial_floats(int rows, int heads, int n_splits) {
    return (long long)n_splits * rows * heads * (R + 4);
}

// rows: rows of the step (padding included); q [rows, heads, D], out [rows, heads, R]; rows that belong to no
// sequence are not written.  max_q_len: an upper bound of q_len over the sequences (sizes the grid).
extern "C" int braid_latent_attn_mma(const void* q, void* out, float* partial, const void* cache, const int* page_table,
                                     const int* q_start, const int* q_len, const int* kv_before, const int* token_seq,
                                     int rows, int n_seqs,
                                     int max_q_len, int heads, int table_cols, int num_pages, int window, int n_splits,
                                     float scale, int* error_flag, void* stream) {
    if (rows <= 0 || n_seqs <= 0 || max_q_len <= 0) return BRAID_OK;
    if (!error_flag) BRAID_REFUSE("latent_attn_mma: error_flag is required");
    if (heads <= 0 || table_cols <= 0 || num_pages <= 0) BRAID_REFUSE("latent_attn_mma: heads=%d, table columns=%d, pages=%d", heads, table_cols, num_pages);
    if (n_splits < 1 || (n_splits > 1 && !partial)) BRAID_REFUSE("latent_attn_mma: %d slices need a workspace", n_splits);
    if (n_splits > LAT_MERGE_MAX_SPLITS) BRAID_REFUSE("latent_attn_mma: at most %d slices, not %d", LAT_MERGE_MAX_SPLITS, n_splits);
    if (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15) BRAID_REFUSE("latent_attn_mma: operands must start on 16 bytes");
    const bool few = braid_latent_attn_tile_rows(max_q_len, heads) == FEW_ROWS;
    const int tile_rows = few ? FEW_ROWS : BM;
    const long long tiles = ((long long)max_q_len * heads + tile_rows - 1) / tile_rows;
    if (tiles > 0x7fffffffLL || n_seqs > 65535 || n_splits * VPARTS > 65535) BRAID_REFUSE("latent_attn_mma: the step exceeds one launch");
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(latent_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess && FEW_OK) e = cudaFuncSetAttribute(latent_attn_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_FEW);
        if (e != cudaSuccess) BRAID_REFUSE("latent_attn_mma: %d bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
        attr_set = true;
    }
    LatAttnArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, n_splits > 1 ? partial : nullptr, (const __nv_bfloat16*)cache,
                  page_table, q_start, q_len, kv_before, heads, table_cols, num_pages, window, n_splits, rows * heads,
                  scale * 1.4426950408889634f, error_flag};
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = few
        ? braid_launch(latent_attn_few_kernel, dim3((unsigned)tiles, n_seqs, n_splits), dim3(128), (size_t)SMEM_FEW, s, a)
        : braid_launch(latent_attn_mma_kernel, dim3((unsigned)tiles, n_seqs, n_splits * VPARTS), dim3(128), (size_t)SMEM_BYTES, s, a);
    if (e == cudaSuccess && n_splits > 1)
        braid_launch(latent_attn_merge_kernel, dim3(rows * heads), dim3(128), 0, s, (const float*)partial, (__nv_bfloat16*)out,
                     token_seq, heads, rows * heads, n_splits);
    BRAID_LAUNCH_CHECK();
}
