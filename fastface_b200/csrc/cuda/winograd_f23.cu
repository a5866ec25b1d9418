// winograd_f23.cu -- exact-integer Winograd F(2,3) convolution on the CUDA cores, kept as the
// measured alternative to the tensor-core implicit GEMM for the 3x3 stride-1 layers.
//
// Same mathematics as the reference's integer Winograd (kernels/winograd_int8_ref.c:14-27,
// 117-179): with G' = 2G the weight transform u = G' g G'^T stays integral (|u| <= 1016, int16),
// the input transform v = B^T d B has |v| <= 508 (int16), and
//   Y' = A^T [ sum_ci u (*) v ] A  =  4 x the direct convolution's int32 accumulator,
// exactly (the reference's self-test checks "== 4 x direct", :237-259).  int16 operands do not
// fit tcgen05.mma kind::i8, so this runs as 16 small integer GEMMs on 32-bit multiply-adds.
//
// Layout of the work: a block owns 16 Winograd tiles (a 4 x 4 group of 2x2 output tiles = 8 x 8
// output pixels of one image) and all output channels.  It stages the 10 x 10 x Cin input patch
// in shared memory, forms v[16][16 tiles][Cin] there, and for each of the 16 transform
// positions multiplies the 16 x Cin slice of v by the Cout x Cin slice of u (streamed from
// global memory, L2-resident).  The output transform is linear, so each position's product is
// added straight into the four outputs of its tile with its +-1 / 0 coefficients: a thread
// carries 4 x 4 output accumulators and never holds the 16 intermediate planes.

#include "ffcu_internal.cuh"

// u[pos][co][ci] = (G' g G'^T)[pos] for every (co, ci); g is OIHW int8.
__global__ void wino_weight_transform_kernel(const int8_t* __restrict__ g, int Cout, int Cin, int16_t* __restrict__ u)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= Cout * Cin) return;
    int a[3][3];
#pragma unroll
    for (int i = 0; i < 3; i++)
#pragma unroll
        for (int j = 0; j < 3; j++) a[i][j] = g[(size_t)idx * 9 + i * 3 + j];
    int t[4][3];
#pragma unroll
    for (int j = 0; j < 3; j++) {
        t[0][j] = 2 * a[0][j];
        t[1][j] = a[0][j] + a[1][j] + a[2][j];
        t[2][j] = a[0][j] - a[1][j] + a[2][j];
        t[3][j] = 2 * a[2][j];
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r[4] = {2 * t[i][0], t[i][0] + t[i][1] + t[i][2], t[i][0] - t[i][1] + t[i][2], 2 * t[i][2]};
#pragma unroll
        for (int j = 0; j < 4; j++) u[(size_t)(i * 4 + j) * Cout * Cin + idx] = (int16_t)r[j];
    }
}

#define WINO_TILES 16        // Winograd tiles per block: 4 x 4 tiles = 8 x 8 output pixels
#define WINO_THREADS 256
#define WINO_PATCH 10        // input pixels per side of the block's patch

// in int8 [B][H][W][Cin] (H, W multiples of 8), u int16 [16][Cout][Cin], out int32 [B][H][W][Cout] = 4 x direct.
// Cin a multiple of 16 and at most 128; Cout a multiple of 64.
__global__ void __launch_bounds__(WINO_THREADS)
wino_f23_kernel(const int8_t* __restrict__ in, const int16_t* __restrict__ u, int H, int W, int Cin, int Cout,
                int32_t* __restrict__ out)
{
    extern __shared__ __align__(16) uint8_t wsm[];
    int8_t* patch = (int8_t*)wsm;                                            // [10][10][Cin]
    int16_t* v = (int16_t*)(wsm + ((WINO_PATCH * WINO_PATCH * Cin + 15) & ~15)); // [16 pos][16 tiles][Cin + 2]
    const int vpitch = Cin + 2;                                              // odd word pitch: tiles hit different banks
    const int bx = blockIdx.x, by = blockIdx.y, b = blockIdx.z;
    const int oh0 = by * 8, ow0 = bx * 8;
    const int8_t* inb = in + (size_t)b * H * W * Cin;

    // ---- stage the input patch (zero padding outside the image), 16 bytes per thread step ----
    const int chunks = Cin / 16;
    for (int i = threadIdx.x; i < WINO_PATCH * WINO_PATCH * chunks; i += WINO_THREADS) {
        const int c = i % chunks, px = (i / chunks) % WINO_PATCH, py = i / (chunks * WINO_PATCH);
        const int ih = oh0 - 1 + py, iw = ow0 - 1 + px;
        int4 val = make_int4(0, 0, 0, 0);
        if (ih >= 0 && ih < H && iw >= 0 && iw < W) val = __ldg((const int4*)(inb + ((size_t)ih * W + iw) * Cin) + c);
        *(int4*)(patch + (py * WINO_PATCH + px) * Cin + c * 16) = val;
    }
    __syncthreads();

    // ---- input transform v = B^T d B per (tile, ci) ----
    for (int i = threadIdx.x; i < WINO_TILES * Cin; i += WINO_THREADS) {
        const int ci = i % Cin, t = i / Cin;
        const int ty = t >> 2, tx = t & 3;
        int d[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) d[r][c] = patch[((2 * ty + r) * WINO_PATCH + 2 * tx + c) * Cin + ci];
        int m[4][4];
#pragma unroll
        for (int c = 0; c < 4; c++) {                     // B^T d
            m[0][c] = d[0][c] - d[2][c];
            m[1][c] = d[1][c] + d[2][c];
            m[2][c] = d[2][c] - d[1][c];
            m[3][c] = d[1][c] - d[3][c];
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {                     // (B^T d) B
            v[((r * 4 + 0) * WINO_TILES + t) * vpitch + ci] = (int16_t)(m[r][0] - m[r][2]);
            v[((r * 4 + 1) * WINO_TILES + t) * vpitch + ci] = (int16_t)(m[r][1] + m[r][2]);
            v[((r * 4 + 2) * WINO_TILES + t) * vpitch + ci] = (int16_t)(m[r][2] - m[r][1]);
            v[((r * 4 + 3) * WINO_TILES + t) * vpitch + ci] = (int16_t)(m[r][1] - m[r][3]);
        }
    }
    __syncthreads();

    // ---- 16 products, accumulated through the output transform ----
    // thread -> (tile, 4 consecutive output channels); Cout / 64 passes over the channel blocks
    const int t = threadIdx.x >> 4;                       // 0..15
    const int cq = threadIdx.x & 15;                      // channel quad within a block of 64
    const int ty = t >> 2, tx = t & 3;
    for (int cb = 0; cb < Cout; cb += 64) {
        const int co = cb + cq * 4;
        int y[4][4];                                      // [channel][2x2 output position]
#pragma unroll
        for (int k = 0; k < 4; k++)
#pragma unroll
            for (int q = 0; q < 4; q++) y[k][q] = 0;
#pragma unroll
        for (int pos = 0; pos < 16; pos++) {
            const int16_t* vp = v + (pos * WINO_TILES + t) * vpitch;
            const int16_t* up = u + ((size_t)pos * Cout + co) * Cin;
            int m[4] = {0, 0, 0, 0};
            for (int ci = 0; ci < Cin; ci += 8) {
                // eight input channels: v from shared memory (4-byte reads), u rows from L2 (16-byte reads)
                int vv[8];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int pr = *(const int*)(vp + ci + 2 * k);
                    vv[2 * k] = (int)(int16_t)(pr & 0xffff); vv[2 * k + 1] = pr >> 16;
                }
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int4 uu = __ldg((const int4*)(up + (size_t)k * Cin + ci));
                    const int w8[8] = {(int)(int16_t)(uu.x & 0xffff), uu.x >> 16, (int)(int16_t)(uu.y & 0xffff), uu.y >> 16,
                                       (int)(int16_t)(uu.z & 0xffff), uu.z >> 16, (int)(int16_t)(uu.w & 0xffff), uu.w >> 16};
#pragma unroll
                    for (int e = 0; e < 8; e++) m[k] += vv[e] * w8[e];
                }
            }
            // Y = A^T M A with A^T = [[1,1,1,0],[0,1,-1,-1]]: position (i, j) feeds output (di, dj)
            // with coefficient at[di][i] * at[dj][j]
            const int i = pos >> 2, j = pos & 3;
            const int ai0 = (i <= 2) ? 1 : 0, ai1 = (i == 1) ? 1 : (i >= 2 ? -1 : 0);
            const int aj0 = (j <= 2) ? 1 : 0, aj1 = (j == 1) ? 1 : (j >= 2 ? -1 : 0);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                y[k][0] += ai0 * aj0 * m[k];
                y[k][1] += ai0 * aj1 * m[k];
                y[k][2] += ai1 * aj0 * m[k];
                y[k][3] += ai1 * aj1 * m[k];
            }
        }
        int32_t* ob = out + (size_t)b * H * W * Cout;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int oh = oh0 + 2 * ty + (q >> 1), ow = ow0 + 2 * tx + (q & 1);
            *(int4*)(ob + ((size_t)oh * W + ow) * Cout + co) = make_int4(y[0][q], y[1][q], y[2][q], y[3][q]);
        }
    }
}

// One 3x3 stride-1 pad-1 convolution by integer Winograd F(2,3) on host tensors: in int8
// [B][H][W][Cin], w int8 OIHW -> out int32 [B][H][W][Cout] = 4 x the direct accumulator.  The
// weight transform runs once (a load-time cost in a deployment); *ms receives the mean CUDA-event
// time of `iters` runs of the convolution kernel alone.
extern "C" int ffcu_winograd_f23_once(int device, const int8_t* in, const int8_t* w_oihw, int B, int H, int W, int Cin,
                                      int Cout, int iters, int32_t* out, float* ms)
{
    if (!in || !w_oihw || !out || B < 1 || iters < 1) { ffcu_set_error("ffcu_winograd_f23_once: bad arguments"); return -1; }
    if (H % 8 || W % 8 || Cin % 16 || Cin > 128 || Cout % 64) {
        ffcu_set_error("ffcu_winograd_f23_once: needs H, W multiples of 8, Cin a multiple of 16 (<= 128), Cout a multiple of 64");
        return -2;
    }
    FFCU_CHECK(cudaSetDevice(device));
    const size_t in_bytes = (size_t)B * H * W * Cin, out_elems = (size_t)B * H * W * Cout, wn = (size_t)Cout * Cin * 9;
    int8_t *d_in = nullptr, *d_w = nullptr; int16_t* d_u = nullptr; int32_t* d_out = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = 0;
    auto ok = [&](cudaError_t e, const char* what) {
        if (e != cudaSuccess && rc == 0) { ffcu_set_error("%s failed: %s", what, cudaGetErrorString(e)); rc = -100; }
        return rc == 0;
    };
    ok(cudaMalloc(&d_in, in_bytes), "cudaMalloc(in)") && ok(cudaMalloc(&d_w, wn), "cudaMalloc(w)") &&
        ok(cudaMalloc(&d_u, 16 * (size_t)Cout * Cin * sizeof(int16_t)), "cudaMalloc(u)") &&
        ok(cudaMalloc(&d_out, out_elems * 4), "cudaMalloc(out)") &&
        ok(cudaMemcpy(d_in, in, in_bytes, cudaMemcpyHostToDevice), "copy in") &&
        ok(cudaMemcpy(d_w, w_oihw, wn, cudaMemcpyHostToDevice), "copy w") &&
        ok(cudaEventCreate(&e0), "event") && ok(cudaEventCreate(&e1), "event");
    const int smem = ((WINO_PATCH * WINO_PATCH * Cin + 15) & ~15) + 16 * WINO_TILES * (Cin + 2) * 2;
    if (rc == 0) {
        wino_weight_transform_kernel<<<(Cout * Cin + 255) / 256, 256>>>(d_w, Cout, Cin, d_u);
        ok(cudaFuncSetAttribute(wino_f23_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "smem attribute");
    }
    if (rc == 0) {
        const dim3 grid(W / 8, H / 8, B);
        wino_f23_kernel<<<grid, WINO_THREADS, smem>>>(d_in, d_u, H, W, Cin, Cout, d_out);      // warm-up, and the result
        ok(cudaEventRecord(e0), "record");
        for (int it = 0; it < iters; it++) wino_f23_kernel<<<grid, WINO_THREADS, smem>>>(d_in, d_u, H, W, Cin, Cout, d_out);
        ok(cudaEventRecord(e1), "record");
        ok(cudaEventSynchronize(e1), "kernel");
        float t = 0;
        if (rc == 0 && ok(cudaEventElapsedTime(&t, e0, e1), "elapsed") && ms) *ms = t / iters;
        ok(cudaMemcpy(out, d_out, out_elems * 4, cudaMemcpyDeviceToHost), "copy out");
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(d_in); cudaFree(d_w); cudaFree(d_u); cudaFree(d_out);
    return rc;
}
