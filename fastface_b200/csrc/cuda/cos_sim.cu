// cos_sim.cu -- cosine-similarity matrix of two sets of 512-d embeddings.
//
// out[i][j] = CosSim(a[i], b[j]) with the arithmetic of the reference's Go wrapper
// (go/fastface/fastface.go:157-168): dot product and both squared norms accumulated in
// float64 in index order, 0 when a norm is 0, result rounded to float32 once at the end.  A
// float32 x float32 product is exact in float64, so "dot += x * y" rounds once per step whether
// or not the compiler fuses it; the kernel therefore reproduces the host function bit for bit.
// One thread per (i, j); a block of 16 x 16 threads stages 16 + 16 embeddings in shared memory
// 64 dimensions at a time (the accumulation order over k is unchanged).
#include "ffcu_internal.cuh"

#define CS_DIM 512
#define CS_T 16
#define CS_KC 64

__global__ void __launch_bounds__(CS_T * CS_T) cos_sim_matrix_kernel(const float* __restrict__ a, int n,
                                                                    const float* __restrict__ b, int m,
                                                                    float* __restrict__ out)
{
    __shared__ float sa[CS_T][CS_KC + 1], sb[CS_T][CS_KC + 1];
    const int tx = threadIdx.x % CS_T, ty = threadIdx.x / CS_T;
    const int i = blockIdx.y * CS_T + ty, j = blockIdx.x * CS_T + tx;
    double dot = 0.0, na = 0.0, nb = 0.0;
    for (int k0 = 0; k0 < CS_DIM; k0 += CS_KC) {
        for (int e = threadIdx.x; e < CS_T * CS_KC; e += CS_T * CS_T) {
            const int r = e / CS_KC, c = e % CS_KC;
            const int ia = blockIdx.y * CS_T + r, jb = blockIdx.x * CS_T + r;
            sa[r][c] = ia < n ? a[(size_t)ia * CS_DIM + k0 + c] : 0.0f;
            sb[r][c] = jb < m ? b[(size_t)jb * CS_DIM + k0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll 8
        for (int c = 0; c < CS_KC; c++) {
            const double x = (double)sa[ty][c], y = (double)sb[tx][c];
            dot = __dadd_rn(dot, __dmul_rn(x, y));
            na = __dadd_rn(na, __dmul_rn(x, x));
            nb = __dadd_rn(nb, __dmul_rn(y, y));
        }
        __syncthreads();
    }
    if (i < n && j < m) {
        float r = 0.0f;
        if (na != 0.0 && nb != 0.0) r = (float)__ddiv_rn(dot, __dmul_rn(__dsqrt_rn(na), __dsqrt_rn(nb)));
        out[(size_t)i * m + j] = r;
    }
}

// a: host [n][512], b: host [m][512], out: host [n][m].  Returns 0 or a negative code.
extern "C" int ffcu_cos_sim_matrix(int device, const float* a, int n, const float* b, int m, float* out)
{
    if (!a || !b || !out || n < 1 || m < 1) { ffcu_set_error("ffcu_cos_sim_matrix: bad arguments"); return -1; }
    FFCU_CHECK(cudaSetDevice(device));
    float *da = nullptr, *db = nullptr, *dout = nullptr;
    int rc = 0;
    if (cudaMalloc(&da, (size_t)n * CS_DIM * 4) != cudaSuccess || cudaMalloc(&db, (size_t)m * CS_DIM * 4) != cudaSuccess ||
        cudaMalloc(&dout, (size_t)n * m * 4) != cudaSuccess) {
        ffcu_set_error("ffcu_cos_sim_matrix: device allocation failed");
        cudaGetLastError();
        rc = -2;
    }
    if (rc == 0) {
        cudaMemcpy(da, a, (size_t)n * CS_DIM * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(db, b, (size_t)m * CS_DIM * 4, cudaMemcpyHostToDevice);
        dim3 grid((m + CS_T - 1) / CS_T, (n + CS_T - 1) / CS_T);
        cos_sim_matrix_kernel<<<grid, CS_T * CS_T>>>(da, n, db, m, dout);
        cudaError_t e = cudaMemcpy(out, dout, (size_t)n * m * 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { ffcu_set_error("ffcu_cos_sim_matrix: %s", cudaGetErrorString(e)); rc = -100; }
    }
    cudaFree(da); cudaFree(db); cudaFree(dout);
    return rc;
}
