// Dense contractions of the multiplicative update, fp32 on the CUDA cores:
//   gram      G[r,r] = X^T X for a tall X [rows, r]       (H*H^T and W^T*W)
//   mu_update X[i,c] *= Num[i,c] / (sum_t X[i,t] G[t,c] + eps)
//             ((W^T W)*H or W*(H H^T), fused with the elementwise update)
// They replace the four cublasSgemm calls per iteration
// (multi_mu_dense_factors_device_contexts1.h:303,306,322,329) and
// kernelNmfMuUpdate (src/nmf/sparse/kernels.h:24-34).
#pragma once
#include "common.cuh"

namespace dnpeff {

// ---------------------------------------------------------------------------
// Gram: the r x r output is cut into TILE x TILE tiles; only tile pairs
// (ti <= tj) are computed.  The rows of X are cut into slabs; block (pair, slab)
// writes one partial tile to scratch; k_gram_reduce adds the slabs in index
// order in double and mirrors the lower triangle.  Fixed order => repeatable.
constexpr int kGramBK = 16;

__host__ __device__ inline int gram_pair_index(int ti, int tj, int ntile) {
    return ti * ntile - ti * (ti - 1) / 2 + (tj - ti);
}

template <int TILE>
__device__ __forceinline__ void gram_load_stage(const float* __restrict__ X, int64_t kb,
                                                int64_t row1, int r, int col0, bool vec_ok,
                                                float (*S)[TILE]) {
    constexpr int PER = TILE * kGramBK / 256;  // floats per thread
    if (vec_ok) {
#pragma unroll
        for (int i = 0; i < PER / 4; i++) {
            int e = threadIdx.x + 256 * i;
            int rr = e / (TILE / 4), c4 = e % (TILE / 4);
            int64_t row = kb + rr;
            int col = col0 + c4 * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < row1 && col < r) v = __ldg((const float4*)(X + row * r + col));
            *(float4*)&S[rr][c4 * 4] = v;
        }
    } else {
#pragma unroll
        for (int i = 0; i < PER; i++) {
            int e = threadIdx.x + 256 * i;
            int rr = e / TILE, c = e % TILE;
            int64_t row = kb + rr;
            int col = col0 + c;
            S[rr][c] = (row < row1 && col < r) ? __ldg(X + row * r + col) : 0.f;
        }
    }
}

template <int TILE>
__global__ void __launch_bounds__(256)
k_gram_partial(const float* __restrict__ X, int64_t rows, int r, int ntile, int64_t rows_per_slab,
               float* __restrict__ partial) {
    constexpr int M = TILE / 16;
    __shared__ __align__(16) float As[kGramBK][TILE];
    __shared__ __align__(16) float Bs[kGramBK][TILE];
    int ti = 0, tj = 0;
    {
        int rem = blockIdx.x;
        for (ti = 0; ti < ntile; ti++) {
            int len = ntile - ti;
            if (rem < len) { tj = ti + rem; break; }
            rem -= len;
        }
    }
    const bool diag = (ti == tj);
    const bool vec_ok = (r % 4) == 0;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int64_t row0 = (int64_t)blockIdx.y * rows_per_slab;
    int64_t row1 = row0 + rows_per_slab < rows ? row0 + rows_per_slab : rows;
    float acc[M][M];
#pragma unroll
    for (int i = 0; i < M; i++)
#pragma unroll
        for (int j = 0; j < M; j++) acc[i][j] = 0.f;

    for (int64_t kb = row0; kb < row1; kb += kGramBK) {
        gram_load_stage<TILE>(X, kb, row1, r, ti * TILE, vec_ok, As);
        if (!diag) gram_load_stage<TILE>(X, kb, row1, r, tj * TILE, vec_ok, Bs);
        __syncthreads();
        float (*Bp)[TILE] = diag ? As : Bs;
#pragma unroll
        for (int kk = 0; kk < kGramBK; kk++) {
            float a[M], b[M];
            if constexpr (M == 8) {
                *(float4*)&a[0] = *(const float4*)&As[kk][ty * 4];
                *(float4*)&a[4] = *(const float4*)&As[kk][TILE / 2 + ty * 4];
                *(float4*)&b[0] = *(const float4*)&Bp[kk][tx * 4];
                *(float4*)&b[4] = *(const float4*)&Bp[kk][TILE / 2 + tx * 4];
            } else {
                *(float4*)&a[0] = *(const float4*)&As[kk][ty * 4];
                *(float4*)&b[0] = *(const float4*)&Bp[kk][tx * 4];
            }
#pragma unroll
            for (int i = 0; i < M; i++)
#pragma unroll
                for (int j = 0; j < M; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* out = partial + ((int64_t)blockIdx.y * gridDim.x + blockIdx.x) * (TILE * TILE);
#pragma unroll
    for (int i = 0; i < M; i++) {
        int ri = (M == 8 && i >= 4) ? (TILE / 2 + ty * 4 + i - 4) : (ty * 4 + i);
#pragma unroll
        for (int j = 0; j < M; j += 4) {
            int cj = (M == 8 && j >= 4) ? (TILE / 2 + tx * 4) : (tx * 4);
            *(float4*)&out[ri * TILE + cj] =
                make_float4(acc[i][j], acc[i][j + 1], acc[i][j + 2], acc[i][j + 3]);
        }
    }
}

// G[a,b] = sum over slabs of the partial tile element, slabs in index order.
static __global__ void k_gram_reduce(const float* __restrict__ partial, int nslab, int npairs, int ntile,
                              int tile, int r, float* __restrict__ G) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= r * r) return;
    int a = idx / r, b = idx % r;
    int ti = a / tile, tj = b / tile, ea = a % tile, eb = b % tile;
    // read the upper triangle only (also inside a diagonal tile), so that the
    // result is symmetric bit for bit whatever computed the tiles
    if (ti > tj || (ti == tj && ea > eb)) {
        int t = ti; ti = tj; tj = t;
        t = ea; ea = eb; eb = t;
    }
    int pair = gram_pair_index(ti, tj, ntile);
    const float* p = partial + (int64_t)pair * (tile * tile) + ea * tile + eb;
    int64_t stride = (int64_t)npairs * (tile * tile);
    double s = 0.0;
    for (int sl = 0; sl < nslab; sl++) s += (double)p[sl * stride];
    G[idx] = (float)s;
}

struct GramPlan {
    int tile, ntile, npairs, nslab;
    int64_t rows_per_slab;
    size_t scratch_floats;
};

inline GramPlan gram_plan(int64_t rows, int r) {
    GramPlan g;
    g.tile = (r > 64) ? 128 : 64;
    g.ntile = (int)ceil_div(r, g.tile);
    g.npairs = g.ntile * (g.ntile + 1) / 2;
    int64_t want = ceil_div(rows > 0 ? rows : 1, 512);
    int64_t cap = (4 * kNumSMs) / g.npairs;  // about 4 blocks per SM over all pairs
    if (cap < 1) cap = 1;
    g.nslab = (int)(want < cap ? want : cap);
    if (g.nslab < 1) g.nslab = 1;
    g.rows_per_slab = ceil_div(rows > 0 ? rows : 1, g.nslab);
    g.rows_per_slab = ceil_div(g.rows_per_slab, kGramBK) * kGramBK;
    g.nslab = (int)ceil_div(rows > 0 ? rows : 1, g.rows_per_slab);
    g.scratch_floats = (size_t)g.nslab * g.npairs * g.tile * g.tile;
    return g;
}

// scratch must hold g.scratch_floats floats.
inline int gram_launch_plan(const float* X, int64_t rows, int r, float* G, float* scratch,
                            const GramPlan& g, cudaStream_t st) {
    dim3 grid(g.npairs, g.nslab);
    if (g.tile == 128)
        k_gram_partial<128><<<grid, 256, 0, st>>>(X, rows, r, g.ntile, g.rows_per_slab, scratch);
    else
        k_gram_partial<64><<<grid, 256, 0, st>>>(X, rows, r, g.ntile, g.rows_per_slab, scratch);
    DN_LAUNCH_CHECK();
    k_gram_reduce<<<(unsigned)ceil_div((int64_t)r * r, 256), 256, 0, st>>>(
        scratch, g.nslab, g.npairs, g.ntile, g.tile, r, G);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(2);
    return DNPEFF_OK;
}

// scratch must hold gram_plan(rows, r).scratch_floats floats.
inline int gram_launch(const float* X, int64_t rows, int r, float* G, float* scratch,
                       cudaStream_t st) {
    return gram_launch_plan(X, rows, r, G, scratch, gram_plan(rows, r), st);
}

// ---------------------------------------------------------------------------
// mu_update: a block owns TR = 16384/RP whole rows of X (RP = r rounded up to
// 32..512).  It first stages its rows, transposed, in shared memory -- after
// that nothing reads those rows from global memory again, so the update can be
// written in place -- then runs a TR x RP x r SGEMM against G streamed in
// 16-row chunks, and finishes with the elementwise rule
//     t = den + eps;  q = num / t;  x = x * q      (kernels.h:31-33 order).
constexpr int kMuKC = 16;

template <int RP>
__global__ void __launch_bounds__(256)
k_mu_update(float* __restrict__ X, const float* __restrict__ Num, const float* __restrict__ G,
            int64_t rows, int r, float eps) {
    constexpr int TR = 16384 / RP;
    constexpr int TX = RP / 8;
    extern __shared__ __align__(16) float smem[];
    float (*XsT)[TR] = (float (*)[TR])smem;                    // [RP][TR]
    float (*Gs)[RP] = (float (*)[RP])(smem + (size_t)RP * TR);  // [kMuKC][RP]
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int r4 = r / 4;
    const int64_t row0 = (int64_t)blockIdx.x * TR;

    // stage X rows transposed: lane <-> row, so the shared stores hit 32 banks
    for (int rg = 0; rg < TR / 32; rg++) {
        int rl = rg * 32 + lane;
        int64_t row = row0 + rl;
        for (int kq = 2 * w; kq < r4; kq += 16) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                int q = kq + h;
                if (q < r4) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (row < rows) v = *(const float4*)(X + row * r + q * 4);
                    XsT[q * 4 + 0][rl] = v.x;
                    XsT[q * 4 + 1][rl] = v.y;
                    XsT[q * 4 + 2][rl] = v.z;
                    XsT[q * 4 + 3][rl] = v.w;
                }
            }
        }
    }

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < r; k0 += kMuKC) {
        __syncthreads();  // X staged (first pass) / previous chunk consumed
        for (int e = threadIdx.x; e < kMuKC * (RP / 4); e += 256) {
            int kk = e / (RP / 4), c4 = e % (RP / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + kk < r && c4 < r4) v = __ldg((const float4*)(G + (int64_t)(k0 + kk) * r + c4 * 4));
            *(float4*)&Gs[kk][c4 * 4] = v;
        }
        __syncthreads();
        int kmax = (r - k0) < kMuKC ? (r - k0) : kMuKC;
#pragma unroll 4
        for (int kk = 0; kk < kmax; kk++) {
            float a[8], b[8];
            *(float4*)&a[0] = *(const float4*)&XsT[k0 + kk][ty * 8];
            *(float4*)&a[4] = *(const float4*)&XsT[k0 + kk][ty * 8 + 4];
            *(float4*)&b[0] = *(const float4*)&Gs[kk][tx * 4];
            *(float4*)&b[4] = *(const float4*)&Gs[kk][RP / 2 + tx * 4];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
    }

#pragma unroll
    for (int i = 0; i < 8; i++) {
        int rl = ty * 8 + i;
        int64_t row = row0 + rl;
        if (row >= rows) continue;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int c = h * (RP / 2) + tx * 4;
            if (c >= r) continue;
            float4 nu = __ldcs((const float4*)(Num + row * r + c));
            float4 o;
            o.x = XsT[c + 0][rl] * __fdiv_rn(nu.x, __fadd_rn(acc[i][h * 4 + 0], eps));
            o.y = XsT[c + 1][rl] * __fdiv_rn(nu.y, __fadd_rn(acc[i][h * 4 + 1], eps));
            o.z = XsT[c + 2][rl] * __fdiv_rn(nu.z, __fadd_rn(acc[i][h * 4 + 2], eps));
            o.w = XsT[c + 3][rl] * __fdiv_rn(nu.w, __fadd_rn(acc[i][h * 4 + 3], eps));
            *(float4*)(X + row * r + c) = o;
        }
    }
}

// Any rank: one warp per row, the row cached in shared memory (r floats per warp).
static __global__ void k_mu_update_generic(float* __restrict__ X, const float* __restrict__ Num,
                                    const float* __restrict__ G, int64_t rows, int r, float eps) {
    extern __shared__ float xs_all[];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float* xs = xs_all + (size_t)w * r;
    int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + w;
    if (row >= rows) return;
    for (int c = lane; c < r; c += 32) xs[c] = X[row * r + c];
    __syncwarp();
    for (int c = lane; c < r; c += 32) {
        float den = 0.f;
        for (int t = 0; t < r; t++) den = fmaf(xs[t], G[(int64_t)t * r + c], den);
        X[row * r + c] = xs[c] * __fdiv_rn(Num[row * r + c], __fadd_rn(den, eps));
    }
}

template <int RP>
inline int mu_update_launch_t(float* X, const float* Num, const float* G, int64_t rows, int r,
                              float eps, cudaStream_t st) {
    constexpr int TR = 16384 / RP;
    size_t smem = ((size_t)RP * TR + (size_t)kMuKC * RP) * sizeof(float);
    // per device, so set on every call rather than once per process
    DN_CUDA(cudaFuncSetAttribute(k_mu_update<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    k_mu_update<RP><<<(unsigned)ceil_div(rows, TR), 256, smem, st>>>(X, Num, G, rows, r, eps);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(1);
    return DNPEFF_OK;
}

inline int mu_update_launch(float* X, const float* Num, const float* G, int64_t rows, int r,
                            float eps, cudaStream_t st) {
    if (rows <= 0) return DNPEFF_OK;
    if (r % 4 == 0 && r <= 512) {
        if (r <= 32) return mu_update_launch_t<32>(X, Num, G, rows, r, eps, st);
        if (r <= 64) return mu_update_launch_t<64>(X, Num, G, rows, r, eps, st);
        if (r <= 128) return mu_update_launch_t<128>(X, Num, G, rows, r, eps, st);
        if (r <= 256) return mu_update_launch_t<256>(X, Num, G, rows, r, eps, st);
        return mu_update_launch_t<512>(X, Num, G, rows, r, eps, st);
    }
    size_t smem = (size_t)8 * r * sizeof(float);
    if (smem > 48 * 1024) return fail(DNPEFF_ERR_UNSUPPORTED, "rank %d too large", r);
    k_mu_update_generic<<<(unsigned)ceil_div(rows, 8), 256, smem, st>>>(X, Num, G, rows, r, eps);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(1);
    return DNPEFF_OK;
}

}  // namespace dnpeff
