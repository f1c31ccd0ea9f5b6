// General matrix product on CUDA cores, any sizes: C = epilogue(A[M,K] · W[N,K]^T).
// Both operands are K-contiguous (W is stored [out][in], the layout of
// src/HyMT2Sharp/HunyuanDenseModel.cs:586-587).  Products and sums are float32
// FMAs in ascending K order, so an output element does not depend on M or on
// its row's place in the batch.  This is the whole of the 32-bit path and the
// fallback of the bfloat16 path for shapes that the tensor-core kernels refuse.
//
// Epilogues:
//   0 store      C = acc
//   1 accumulate C += acc                      (projection back into the residual stream)
//   2 swiglu     C = silu(acc_gate) * acc_up   (W holds N gate rows, then N up rows;
//                                               src/HyMT2Sharp/Ops.cs:1053)
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

enum { EPI_STORE = 0, EPI_ACCUMULATE = 1, EPI_SWIGLU = 2 };

template <typename T>
__device__ __forceinline__ void load4(const T* row, int k, int K, bool row_ok, bool vec, float out[4]) {
    if (row_ok && vec && k + 4 <= K) {
        if constexpr (sizeof(T) == 4) {
            float4 v = *reinterpret_cast<const float4*>(row + k);
            out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
        } else {
            uint2 v = *reinterpret_cast<const uint2*>(row + k);
            __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v.x);
            __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v.y);
            out[0] = __low2float(a); out[1] = __high2float(a); out[2] = __low2float(b); out[3] = __high2float(b);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) out[i] = (row_ok && k + i < K) ? to_float(row[k + i]) : 0.f;
    }
}

template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W, int M, int N, int K,
                 long lda, long ldw, long ldc, bool vec_a, bool vec_w, long a_bs, long w_bs, long c_bs) {
    constexpr int NB = EPI == EPI_SWIGLU ? 2 : 1;
    // a batch of products with the same sizes: blockIdx.z picks the operands (strides in elements)
    A += (size_t)blockIdx.z * a_bs;
    W += (size_t)blockIdx.z * w_bs;
    C += (size_t)blockIdx.z * c_bs;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[NB][BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;  // loader: 64 rows x 4 groups of 4 k
    const int tm = (tid >> 4) * TM, tn = (tid & 15) * TN;

    float acc[NB][TM][TN];
#pragma unroll
    for (int b = 0; b < NB; b++)
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
            for (int j = 0; j < TN; j++) acc[b][i][j] = 0.f;

    const bool a_ok = m0 + lrow < M, w_ok = n0 + lrow < N;
    const TA* a_row = A + (size_t)(a_ok ? m0 + lrow : 0) * lda;
    const TW* w_row[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) w_row[b] = W + ((size_t)b * N + (w_ok ? n0 + lrow : 0)) * ldw;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float va[4], vw[NB][4];
        load4(a_row, k0 + lk, K, a_ok, vec_a, va);
#pragma unroll
        for (int b = 0; b < NB; b++) load4(w_row[b], k0 + lk, K, w_ok, vec_w, vw[b]);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            As[lk + i][lrow] = va[i];
#pragma unroll
            for (int b = 0; b < NB; b++) Ws[b][lk + i][lrow] = vw[b][i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], w[NB][TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][tm + i];
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int j = 0; j < TN; j++) w[b][j] = Ws[b][kk][tn + j];
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int i = 0; i < TM; i++)
#pragma unroll
                    for (int j = 0; j < TN; j++) acc[b][i][j] = fmaf(a[i], w[b][j], acc[b][i][j]);
        }
    }

#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tn + j;
            if (n >= N) continue;
            TC* c = C + (size_t)m * ldc + n;
            if constexpr (EPI == EPI_STORE) {
                *c = from_float<TC>(acc[0][i][j]);
            } else if constexpr (EPI == EPI_ACCUMULATE) {
                *c = from_float<TC>(to_float(*c) + acc[0][i][j]);
            } else {
                const float g = acc[0][i][j], u = acc[NB - 1][i][j];
                *c = from_float<TC>(g / (1.0f + expf(-g)) * u);
            }
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(void* C, const void* A, const void* W, int M, int N, int K, long lda, long ldw, long ldc, int epi,
           cudaStream_t stream, int batch = 1, long a_bs = 0, long w_bs = 0, long c_bs = 0) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    const bool vec_a = (lda % 4 == 0) && ((uintptr_t)A % 16 == 0) && (a_bs * sizeof(TA)) % 16 == 0;
    const bool vec_w = (ldw % 4 == 0) && ((uintptr_t)W % 16 == 0) && (w_bs * sizeof(TW)) % 16 == 0;
#define HYMT2_GEMM_CASE(E)                                                                                  \
    gemm_simt_kernel<TA, TW, TC, E><<<grid, THREADS, 0, stream>>>((TC*)C, (const TA*)A, (const TW*)W, M, N, K, \
                                                                  lda, ldw, ldc, vec_a, vec_w, a_bs, w_bs, c_bs)
    if (epi == EPI_STORE) HYMT2_GEMM_CASE(EPI_STORE);
    else if (epi == EPI_ACCUMULATE) HYMT2_GEMM_CASE(EPI_ACCUMULATE);
    else HYMT2_GEMM_CASE(EPI_SWIGLU);
#undef HYMT2_GEMM_CASE
    return hymt2_check_launch("gemm_simt");
}


// A grouped product: the rows of A are sorted by the matrix they meet (an expert of a mixture), in segments padded to whole
// tiles of BM rows.  `tile_group[i]` names the matrix of row tile i (-1: the tile is not in use), `row_source[r]` the row of
// A that sorted row r reads (-1: a padding row; with `gather` 0 it only says which rows are in use, and sorted row r reads
// row r of A).  C has one row per sorted row.  Epilogues: 0 store,
// 3 the square of relu.  Sums run in ascending K as everywhere, so a row's result depends on nothing but the row.
enum { EPI_RELU_SQUARED = 3 };

template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_simt_grouped_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W, const int* __restrict__ tile_group,
                         const int* __restrict__ row_source, int gather, int N, int K, long lda, long ldc, long w_gs, bool vec_a,
                         bool vec_w) {
    pdl_wait();
    pdl_launch_dependents();
    const int group = tile_group[blockIdx.y];
    if (group < 0) return;
    W += (size_t)group * w_gs;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int rows_ok[BM];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const int tm = (tid >> 4) * TM, tn = (tid & 15) * TN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;
    int src_row = row_source ? row_source[m0 + lrow] : m0 + lrow;
    if ((tid & 3) == 0) rows_ok[lrow] = src_row >= 0;
    if (!gather && src_row >= 0) src_row = m0 + lrow;
    const bool a_ok = src_row >= 0, w_ok = n0 + lrow < N;
    const TA* a_row = A + (size_t)(a_ok ? src_row : 0) * lda;
    const TW* w_row = W + (size_t)(w_ok ? n0 + lrow : 0) * K;
    for (int k0 = 0; k0 < K; k0 += BK) {
        float va[4], vw[4];
        load4(a_row, k0 + lk, K, a_ok, vec_a, va);
        load4(w_row, k0 + lk, K, w_ok, vec_w, vw);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            As[lk + i][lrow] = va[i];
            Ws[lk + i][lrow] = vw[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][tm + i];
#pragma unroll
            for (int j = 0; j < TN; j++) w[j] = Ws[kk][tn + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        if (!rows_ok[tm + i]) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tn + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if constexpr (EPI == EPI_RELU_SQUARED) { v = fmaxf(v, 0.f); v = v * v; }
            C[(size_t)(m0 + tm + i) * ldc + n] = from_float<TC>(v);
        }
    }
}

// Few rows (a decode step's tokens) against a batch of small matrices: one warp per output column reads its weight
// row once, 16 bytes a lane, and keeps a float32 sum for every row of A; the sums of a row do not depend on how many
// other rows there are.  The time is that of reading W once.
constexpr int SKINNY_MAX_ROWS = 16, SKINNY_WARPS = 8;

template <typename T, typename TC>
__global__ void __launch_bounds__(SKINNY_WARPS * 32)
gemm_skinny_batched_kernel(TC* __restrict__ C, const T* __restrict__ A, const T* __restrict__ W, int M, int N, int K,
                           long lda, long ldc, long a_bs, long w_bs, long c_bs, bool vec) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * SKINNY_WARPS + warp;
    if (n >= N) return;
    A += (size_t)blockIdx.y * a_bs;
    C += (size_t)blockIdx.y * c_bs;
    const T* w = W + (size_t)blockIdx.y * w_bs + (size_t)n * K;
    float acc[SKINNY_MAX_ROWS];
#pragma unroll
    for (int m = 0; m < SKINNY_MAX_ROWS; m++) acc[m] = 0.f;
    constexpr int V = 16 / sizeof(T);
    if (vec) {
        for (int k = lane * V; k < K; k += 32 * V) {
            float wv[V];
            const uint4 raw = *reinterpret_cast<const uint4*>(w + k);
            const T* wt = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < V; i++) wv[i] = to_float(wt[i]);
#pragma unroll
            for (int m = 0; m < SKINNY_MAX_ROWS; m++) {
                if (m < M) {
                    const uint4 ra = *reinterpret_cast<const uint4*>(A + (size_t)m * lda + k);
                    const T* at = reinterpret_cast<const T*>(&ra);
#pragma unroll
                    for (int i = 0; i < V; i++) acc[m] = fmaf(to_float(at[i]), wv[i], acc[m]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = to_float(w[k]);
#pragma unroll
            for (int m = 0; m < SKINNY_MAX_ROWS; m++)
                if (m < M) acc[m] = fmaf(to_float(A[(size_t)m * lda + k]), wv, acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < SKINNY_MAX_ROWS; m++) {
        if (m < M) {
            const float v = warp_sum(acc[m]);
            if (lane == 0) C[(size_t)m * ldc + n] = from_float<TC>(v);
        }
    }
}

// The grouped product for few sorted rows (a decode step): row tiles of GROUP_SKINNY_ROWS rows, a warp per output column
// reads its weight row once, 16 bytes a lane, and keeps a float32 sum for every row of the tile.  The time is that of
// reading the matrices of the groups in use once.
constexpr int GROUP_SKINNY_ROWS = 8, GROUP_SKINNY_COLS = 2;   // rows of a tile; output columns (weight rows) of a warp

template <typename T, typename TC, int EPI>
__global__ void __launch_bounds__(SKINNY_WARPS * 32)
gemm_skinny_grouped_kernel(TC* __restrict__ C, const T* __restrict__ A, const T* __restrict__ W, const int* __restrict__ tile_group,
                           const int* __restrict__ row_source, int gather, int N, int K, long lda, long ldc, long w_gs, bool vec) {
    pdl_wait();
    pdl_launch_dependents();
    const int group = tile_group[blockIdx.y];
    if (group < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int COLS = GROUP_SKINNY_COLS;
    const int n0 = (blockIdx.x * SKINNY_WARPS + warp) * COLS;
    if (n0 >= N) return;
    const int m0 = blockIdx.y * GROUP_SKINNY_ROWS;
    const T* a_row[GROUP_SKINNY_ROWS];
    bool ok[GROUP_SKINNY_ROWS];
#pragma unroll
    for (int m = 0; m < GROUP_SKINNY_ROWS; m++) {
        const int src = row_source[m0 + m];
        ok[m] = src >= 0;
        a_row[m] = A + (size_t)(ok[m] ? (gather ? src : m0 + m) : 0) * lda;
    }
    const T* w[COLS];
#pragma unroll
    for (int c = 0; c < COLS; c++) w[c] = W + (size_t)group * w_gs + (size_t)(n0 + c < N ? n0 + c : n0) * K;
    float acc[COLS][GROUP_SKINNY_ROWS];
#pragma unroll
    for (int c = 0; c < COLS; c++)
#pragma unroll
        for (int m = 0; m < GROUP_SKINNY_ROWS; m++) acc[c][m] = 0.f;
    constexpr int V = 16 / sizeof(T);
    if (vec) {
        // four pieces of each weight row in flight per lane: the kernel's time is the weights' way from memory
        constexpr int U = 4;
        for (int k0 = lane * V; k0 < K; k0 += 32 * V * U) {
            uint4 raw[U][COLS];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int k = k0 + u * 32 * V;
#pragma unroll
                for (int c = 0; c < COLS; c++)
                    raw[u][c] = k < K ? __ldg(reinterpret_cast<const uint4*>(w[c] + k)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int k = k0 + u * 32 * V;
                if (k >= K) break;
                float wv[COLS][V];
#pragma unroll
                for (int c = 0; c < COLS; c++) {
                    const T* wt = reinterpret_cast<const T*>(&raw[u][c]);
#pragma unroll
                    for (int i = 0; i < V; i++) wv[c][i] = to_float(wt[i]);
                }
#pragma unroll
                for (int m = 0; m < GROUP_SKINNY_ROWS; m++) {
                    if (ok[m]) {
                        const uint4 ra = *reinterpret_cast<const uint4*>(a_row[m] + k);
                        const T* at = reinterpret_cast<const T*>(&ra);
#pragma unroll
                        for (int i = 0; i < V; i++) {
                            const float av = to_float(at[i]);
#pragma unroll
                            for (int c = 0; c < COLS; c++) acc[c][m] = fmaf(av, wv[c][i], acc[c][m]);
                        }
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            float wv[COLS];
#pragma unroll
            for (int c = 0; c < COLS; c++) wv[c] = to_float(w[c][k]);
#pragma unroll
            for (int m = 0; m < GROUP_SKINNY_ROWS; m++)
                if (ok[m]) {
                    const float av = to_float(a_row[m][k]);
#pragma unroll
                    for (int c = 0; c < COLS; c++) acc[c][m] = fmaf(av, wv[c], acc[c][m]);
                }
        }
    }
#pragma unroll
    for (int m = 0; m < GROUP_SKINNY_ROWS; m++) {
        if (ok[m]) {
#pragma unroll
            for (int c = 0; c < COLS; c++) {
                float v = warp_sum(acc[c][m]);
                if constexpr (EPI == EPI_RELU_SQUARED) { v = fmaxf(v, 0.f); v = v * v; }
                if (lane == 0 && n0 + c < N) C[(size_t)(m0 + m) * ldc + n0 + c] = from_float<TC>(v);
            }
        }
    }
}

}  // namespace

// C[M,N] (ldc) = epilogue(A[M,K] (lda) · W[N,K]^T (ldw)); for the swiglu epilogue W has 2N rows.
HYMT2_API int hymt2_gemm_simt(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype,
                              int M, int N, int K, long lda, long ldw, long ldc, int epilogue,
                              cudaStream_t stream) {
    if (M == 0 || N == 0) return HYMT2_OK;
    HYMT2_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    HYMT2_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm: unknown epilogue %d", epilogue);
    HYMT2_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: a leading dimension is smaller than its row");
    HYMT2_REQUIRE((M + BM - 1) / BM <= 65535, "gemm: M=%d needs more than 65535 row tiles", M);
    HYMT2_DISPATCH_DTYPE(a_dtype, TA, HYMT2_DISPATCH_DTYPE(w_dtype, TW, HYMT2_DISPATCH_DTYPE(c_dtype, TC,
        return (launch<TA, TW, TC>(C, A, W, M, N, K, lda, ldw, ldc, epilogue, stream)))));
    return HYMT2_OK;
}

// `batch` products of the same sizes in one launch: product z reads A + z * a_bs and W + z * w_bs and writes
// C + z * c_bs (strides in elements).  Per-head and per-block matrices (a block-diagonal gate, a projection that
// every head has of its own) are batches of this kind.
HYMT2_API int hymt2_gemm_simt_batched(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype,
                                      int M, int N, int K, long lda, long ldw, long ldc, int batch, long a_bs,
                                      long w_bs, long c_bs, int epilogue, cudaStream_t stream) {
    if (M == 0 || N == 0 || batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(M > 0 && N > 0 && K > 0 && batch > 0 && batch <= 65535, "gemm: bad sizes M=%d N=%d K=%d batch=%d", M, N, K, batch);
    HYMT2_REQUIRE(epilogue >= 0 && epilogue <= 1, "gemm: a batch takes the store and accumulate epilogues, not %d", epilogue);
    HYMT2_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: a leading dimension is smaller than its row");
    HYMT2_REQUIRE((M + BM - 1) / BM <= 65535, "gemm: M=%d needs more than 65535 row tiles", M);
    HYMT2_DISPATCH_DTYPE(a_dtype, TA, HYMT2_DISPATCH_DTYPE(w_dtype, TW, HYMT2_DISPATCH_DTYPE(c_dtype, TC,
        return (launch<TA, TW, TC>(C, A, W, M, N, K, lda, ldw, ldc, epilogue, stream, batch, a_bs, w_bs, c_bs)))));
    return HYMT2_OK;
}

// The same batch for at most 16 rows of A, A and W of one type (see gemm_skinny_batched_kernel): store epilogue only.
HYMT2_API int hymt2_gemm_skinny_batched(void* C, int c_dtype, const void* A, const void* W, int dtype, int M, int N, int K,
                                        long lda, long ldc, int batch, long a_bs, long w_bs, long c_bs, cudaStream_t stream) {
    if (M == 0 || N == 0 || batch == 0) return HYMT2_OK;
    HYMT2_REQUIRE(M > 0 && M <= SKINNY_MAX_ROWS && N > 0 && K > 0 && batch > 0 && batch <= 65535, "gemm_skinny: bad sizes M=%d N=%d K=%d batch=%d", M, N, K, batch);
    HYMT2_REQUIRE(lda >= K && ldc >= N, "gemm_skinny: a leading dimension is smaller than its row");
    const dim3 grid((N + SKINNY_WARPS - 1) / SKINNY_WARPS, batch);
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        const long v = 16 / sizeof(T);
        const bool vec = K % v == 0 && lda % v == 0 && a_bs % v == 0 && w_bs % v == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0;
        HYMT2_DISPATCH_DTYPE(c_dtype, TC, launch_pdl(gemm_skinny_batched_kernel<T, TC>, grid, dim3(SKINNY_WARPS * 32), 0, stream, (TC*)C,
                                                     (const T*)A, (const T*)W, M, N, K, lda, ldc, a_bs, w_bs, c_bs, vec));
    });
    return hymt2_check_launch("gemm_skinny_batched");
}

// The grouped product (see gemm_simt_grouped_kernel): `tiles` row tiles of 64 sorted rows, W holds the groups' matrices
// [N, K] one after the other (w_gs elements apart).
HYMT2_API int hymt2_gemm_simt_grouped(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype,
                                      const int* tile_group, const int* row_source, int gather, int tiles, int N, int K, long lda, long ldc,
                                      long w_gs, int epilogue, cudaStream_t stream) {
    if (tiles == 0 || N == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tiles > 0 && tiles <= 65535 && N > 0 && K > 0, "gemm_grouped: bad sizes tiles=%d N=%d K=%d", tiles, N, K);
    HYMT2_REQUIRE(epilogue == EPI_STORE || epilogue == EPI_RELU_SQUARED, "gemm_grouped: unknown epilogue %d", epilogue);
    HYMT2_REQUIRE(lda >= K && ldc >= N && tile_group, "gemm_grouped: bad arguments");
    const dim3 grid((N + BN - 1) / BN, tiles);
    HYMT2_DISPATCH_DTYPE(a_dtype, TA, HYMT2_DISPATCH_DTYPE(w_dtype, TW, HYMT2_DISPATCH_DTYPE(c_dtype, TC, {
        const bool vec_a = (lda % 4 == 0) && ((uintptr_t)A % 16 == 0);
        const bool vec_w = (K % 4 == 0) && ((uintptr_t)W % 16 == 0) && (w_gs * sizeof(TW)) % 16 == 0;
        if (epilogue == EPI_STORE)
            launch_pdl(gemm_simt_grouped_kernel<TA, TW, TC, EPI_STORE>, grid, dim3(THREADS), 0, stream, (TC*)C, (const TA*)A, (const TW*)W,
                       tile_group, row_source, gather, N, K, lda, ldc, w_gs, vec_a, vec_w);
        else
            launch_pdl(gemm_simt_grouped_kernel<TA, TW, TC, EPI_RELU_SQUARED>, grid, dim3(THREADS), 0, stream, (TC*)C, (const TA*)A,
                       (const TW*)W, tile_group, row_source, gather, N, K, lda, ldc, w_gs, vec_a, vec_w);
    })));
    return hymt2_check_launch("gemm_simt_grouped");
}

HYMT2_API int hymt2_gemm_simt_group_tile() { return BM; }

// The grouped product for few rows: row tiles of hymt2_gemm_skinny_group_tile() sorted rows, A and W of one type.
HYMT2_API int hymt2_gemm_skinny_grouped(void* C, int c_dtype, const void* A, const void* W, int dtype, const int* tile_group,
                                        const int* row_source, int gather, int tiles, int N, int K, long lda, long ldc, long w_gs,
                                        int epilogue, cudaStream_t stream) {
    if (tiles == 0 || N == 0) return HYMT2_OK;
    HYMT2_REQUIRE(tiles > 0 && tiles <= 65535 && N > 0 && K > 0, "gemm_skinny_grouped: bad sizes tiles=%d N=%d K=%d", tiles, N, K);
    HYMT2_REQUIRE(epilogue == EPI_STORE || epilogue == EPI_RELU_SQUARED, "gemm_skinny_grouped: unknown epilogue %d", epilogue);
    HYMT2_REQUIRE(lda >= K && ldc >= N && tile_group && row_source, "gemm_skinny_grouped: bad arguments");
    const int per_block = SKINNY_WARPS * GROUP_SKINNY_COLS;
    const dim3 grid((N + per_block - 1) / per_block, tiles);
    HYMT2_DISPATCH_DTYPE(dtype, T, {
        const long v = 16 / sizeof(T);
        const bool vec = K % v == 0 && lda % v == 0 && w_gs % v == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0;
        HYMT2_DISPATCH_DTYPE(c_dtype, TC, {
            if (epilogue == EPI_STORE)
                launch_pdl(gemm_skinny_grouped_kernel<T, TC, EPI_STORE>, grid, dim3(SKINNY_WARPS * 32), 0, stream, (TC*)C, (const T*)A,
                           (const T*)W, tile_group, row_source, gather, N, K, lda, ldc, w_gs, vec);
            else
                launch_pdl(gemm_skinny_grouped_kernel<T, TC, EPI_RELU_SQUARED>, grid, dim3(SKINNY_WARPS * 32), 0, stream, (TC*)C,
                           (const T*)A, (const T*)W, tile_group, row_source, gather, N, K, lda, ldc, w_gs, vec);
        });
    });
    return hymt2_check_launch("gemm_skinny_grouped");
}

HYMT2_API int hymt2_gemm_skinny_group_tile() { return GROUP_SKINNY_ROWS; }
