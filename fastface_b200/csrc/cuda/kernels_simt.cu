// kernels_simt.cu -- CUDA-core kernels: input quantisation, the stem / generic
// direct convolution (dp4a), the standalone BN pass and the small-batch FC.
//
// These are bandwidth- or latency-bound steps (or, for the generic conv, the
// path for shapes the tensor-core kernel does not take: Cin = 3).

#include "ffcu_internal.cuh"

// ---------------------------------------------------------------------------
// fp32 HWC input -> int8, per channel, ties-to-even
// (reference kernels/int8_epilogue.c:231-247: lrintf(x * inv[c]) then clamp).
// Output pixels are stored as 4 bytes (c0,c1,c2,0) so a pixel is one word.
// ---------------------------------------------------------------------------
__global__ void quant_input_kernel(const float* __restrict__ in, long n_pix,
                                   const float* __restrict__ inv3, int* __restrict__ out)
{
    long p = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pix) return;
    float i0 = __ldg(inv3), i1 = __ldg(inv3 + 1), i2 = __ldg(inv3 + 2);
    const float* x = in + p * 3;
    int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(x[0], i0))));
    int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(x[1], i1))));
    int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(x[2], i2))));
    out[p] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16);
}

int ffcu_launch_quant(const float* in, int n_pix, const float* inv3, int8_t* out4, cudaStream_t s)
{
    int threads = 256;
    long blocks = ((long)n_pix + threads - 1) / threads;
    quant_input_kernel<<<(unsigned)blocks, threads, 0, s>>>(in, n_pix, inv3, (int*)out4);
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// Direct convolution on CUDA cores: exact int8 x int8 -> int32 (dp4a), then the
// fused epilogue.  One thread = one output pixel x 4 consecutive output channels.
//   in  [B][H][W][Cp]   (Cp = Cin rounded up to 4, pad channels are zero)
//   w   [Cout][Kh][Kw][Cp]
//   out [B][Ho][Wo][Cout]
// Takes over fastface_conv2d_i8_nhwc_batched + fused_epilogue_int8
// (reference kernels/conv2d_nhwc.c:179-220, kernels/int8_epilogue.c:25-112).
// ---------------------------------------------------------------------------
template <bool CONTRACT>
__global__ void conv_simt_kernel(const int8_t* __restrict__ in, const int8_t* __restrict__ w,
                                 EpiTables t, const int8_t* __restrict__ res,
                                 int32_t* __restrict__ acc_out, int8_t* __restrict__ out,
                                 int8_t* __restrict__ out_bn2,
                                 int B, int H, int W, int Cp, int Cout, int Kh, int Kw,
                                 int stride, int pad, int Ho, int Wo)
{
    const int cg_per_pix = Cout >> 2;
    long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
    long total = (long)B * Ho * Wo * cg_per_pix;
    if (gid >= total) return;
    int cg = (int)(gid % cg_per_pix);
    long pix = gid / cg_per_pix;
    int ow = (int)(pix % Wo);
    int oh = (int)((pix / Wo) % Ho);
    int b = (int)(pix / ((long)Wo * Ho));
    const int co = cg * 4;
    const int c4n = Cp >> 2;
    const int krow = Kh * Kw * c4n;                 // words per output channel
    const int* w0 = (const int*)w + (long)co * krow;
    int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    for (int kh = 0; kh < Kh; kh++) {
        int ih = oh * stride - pad + kh;
        if (ih < 0 || ih >= H) continue;
        for (int kw = 0; kw < Kw; kw++) {
            int iw = ow * stride - pad + kw;
            if (iw < 0 || iw >= W) continue;
            const int* ip = (const int*)in + (((long)b * H + ih) * W + iw) * c4n;
            const int* wp = w0 + (kh * Kw + kw) * c4n;
            for (int c = 0; c < c4n; c++) {
                int a = __ldg(ip + c);
                a0 = __dp4a(a, __ldg(wp + c), a0);
                a1 = __dp4a(a, __ldg(wp + krow + c), a1);
                a2 = __dp4a(a, __ldg(wp + 2 * krow + c), a2);
                a3 = __dp4a(a, __ldg(wp + 3 * krow + c), a3);
            }
        }
    }
    long o = pix * Cout + co;
    if (acc_out) *(int4*)(acc_out + o) = make_int4(a0, a1, a2, a3);
    if (!out) return;
    int acc[4] = {a0, a1, a2, a3};
    int rw = 0;
    const bool has_res = (res != nullptr) && (t.res_scale != nullptr);
    if (has_res) rw = *(const int*)(res + o);
    unsigned packed = 0, packed2 = 0;
    const bool has_bn2 = (out_bn2 != nullptr) && (t.bn_in != nullptr);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        int c = co + j;
        int r = (int)(int8_t)((rw >> (8 * j)) & 0xff);
        float v = ffcu_conv_fp<CONTRACT>(acc[j], __ldg(t.w_scale + c), __ldg(t.bias + c), has_res, r,
                                         has_res ? __ldg(t.res_scale + c) : 0.0f,
                                         t.slope != nullptr, t.slope ? __ldg(t.slope + c) : 0.0f);
        int q = ffcu_requant(v, __ldg(t.inv_out + c));
        packed |= (unsigned)(q & 0xff) << (8 * j);
        if (has_bn2) {
            int q2 = ffcu_bn_q(q, __ldg(t.bn_in + c), __ldg(t.bn_scale + c), __ldg(t.bn_offset + c), __ldg(t.bn_inv + c));
            packed2 |= (unsigned)(q2 & 0xff) << (8 * j);
        }
    }
    *(unsigned*)(out + o) = packed;
    if (has_bn2) *(unsigned*)(out_bn2 + o) = packed2;
}

int ffcu_launch_conv_simt(const ffcu_layer& L, int batch, int mode, const int8_t* in, const int8_t* w,
                          const EpiTables& t, const int8_t* res, int32_t* acc_out, int8_t* out,
                          int8_t* out_bn2, cudaStream_t s)
{
    long total = (long)batch * L.Ho * L.Wo * (L.Cout / 4);
    int threads = 256;
    long blocks = (total + threads - 1) / threads;
    if (mode)
        conv_simt_kernel<true><<<(unsigned)blocks, threads, 0, s>>>(in, w, t, res, acc_out, out, out_bn2, batch, L.H, L.W,
            L.Cin_pad, L.Cout, L.Kh, L.Kw, L.stride, L.pad, L.Ho, L.Wo);
    else
        conv_simt_kernel<false><<<(unsigned)blocks, threads, 0, s>>>(in, w, t, res, acc_out, out, out_bn2, batch, L.H, L.W,
            L.Cin_pad, L.Cout, L.Kh, L.Kw, L.stride, L.pad, L.Ho, L.Wo);
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// Standalone BN + requant (reference kernels/int8_epilogue.c:253-318).
// One thread = 16 consecutive channels of one position (C is a multiple of 16).
// ---------------------------------------------------------------------------
__global__ void bn_kernel(const int4* __restrict__ in, int4* __restrict__ out, long n_vec, int c16,
                          const float* __restrict__ in_scale, const float* __restrict__ bn_scale,
                          const float* __restrict__ bn_offset, const float* __restrict__ inv_out)
{
    long v = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n_vec) return;
    int c0 = (int)(v % c16) * 16;
    int4 x = in[v];
    int xs[4] = {x.x, x.y, x.z, x.w};
    int ys[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        unsigned packed = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int c = c0 + k * 4 + j;
            int a = (int)(int8_t)((xs[k] >> (8 * j)) & 0xff);
            int q = ffcu_bn_q(a, __ldg(in_scale + c), __ldg(bn_scale + c), __ldg(bn_offset + c), __ldg(inv_out + c));
            packed |= (unsigned)(q & 0xff) << (8 * j);
        }
        ys[k] = (int)packed;
    }
    out[v] = make_int4(ys[0], ys[1], ys[2], ys[3]);
}

int ffcu_launch_bn(const int8_t* in, int8_t* out, size_t n_pos, int C, const float* in_scale,
                   const float* bn_scale, const float* bn_offset, const float* inv_out, cudaStream_t s)
{
    if (C % 16 != 0) { ffcu_set_error("BN kernel needs C %% 16 == 0 (C=%d)", C); return -1; }
    long n_vec = (long)n_pos * (C / 16);
    int threads = 256;
    long blocks = (n_vec + threads - 1) / threads;
    bn_kernel<<<(unsigned)blocks, threads, 0, s>>>((const int4*)in, (int4*)out, n_vec, C / 16,
                                                   in_scale, bn_scale, bn_offset, inv_out);
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// FC on CUDA cores: out[b][n] = bias[n] + (float)dot(act[b], w[n]) * w_scale[n]
// (reference kernels/gemm_int8_matvec.c:33-81).  A block owns 8 outputs x 8 faces;
// its 256 threads split K in 16-byte steps, then reduce.
// ---------------------------------------------------------------------------
#define FC_TN 8
#define FC_TB 8
template <bool CONTRACT>
__global__ void __launch_bounds__(256) fc_simt_kernel(const int8_t* __restrict__ act, const int8_t* __restrict__ w,
                                                      const float* __restrict__ w_scale, const float* __restrict__ bias,
                                                      int B, int N, int K, float* __restrict__ out)
{
    __shared__ int red[8][FC_TB * FC_TN];
    const int n0 = blockIdx.x * FC_TN;
    const int b0 = blockIdx.y * FC_TB;
    int acc[FC_TB][FC_TN];
#pragma unroll
    for (int i = 0; i < FC_TB; i++)
#pragma unroll
        for (int j = 0; j < FC_TN; j++) acc[i][j] = 0;
    const int kv = K >> 4;
    for (int k = threadIdx.x; k < kv; k += blockDim.x) {
        int4 a[FC_TB], ww[FC_TN];
#pragma unroll
        for (int i = 0; i < FC_TB; i++) {
            int b = min(b0 + i, B - 1);
            a[i] = __ldg((const int4*)(act + (size_t)b * K) + k);
        }
#pragma unroll
        for (int j = 0; j < FC_TN; j++) ww[j] = __ldg((const int4*)(w + (size_t)(n0 + j) * K) + k);
#pragma unroll
        for (int i = 0; i < FC_TB; i++)
#pragma unroll
            for (int j = 0; j < FC_TN; j++) {
                int s = acc[i][j];
                s = __dp4a(a[i].x, ww[j].x, s); s = __dp4a(a[i].y, ww[j].y, s);
                s = __dp4a(a[i].z, ww[j].z, s); s = __dp4a(a[i].w, ww[j].w, s);
                acc[i][j] = s;
            }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < FC_TB; i++)
#pragma unroll
        for (int j = 0; j < FC_TN; j++) {
            int s = acc[i][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) red[warp][i * FC_TN + j] = s;
        }
    __syncthreads();
    if (threadIdx.x < FC_TB * FC_TN) {
        int s = 0;
#pragma unroll
        for (int wv = 0; wv < 8; wv++) s += red[wv][threadIdx.x];
        int i = threadIdx.x / FC_TN, j = threadIdx.x % FC_TN;
        int b = b0 + i, n = n0 + j;
        if (b < B) out[(size_t)b * N + n] = ffcu_fc_fp<CONTRACT>(s, __ldg(w_scale + n), __ldg(bias + n));
    }
}

int ffcu_launch_fc_simt(const int8_t* act, const int8_t* w, const float* w_scale, const float* bias,
                        int batch, int N, int K, int mode, float* out, cudaStream_t s)
{
    if (N % FC_TN != 0 || K % 16 != 0) { ffcu_set_error("FC kernel needs N %% 8 == 0 and K %% 16 == 0"); return -1; }
    dim3 grid(N / FC_TN, (batch + FC_TB - 1) / FC_TB);
    if (mode) fc_simt_kernel<true><<<grid, 256, 0, s>>>(act, w, w_scale, bias, batch, N, K, out);
    else      fc_simt_kernel<false><<<grid, 256, 0, s>>>(act, w, w_scale, bias, batch, N, K, out);
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// Fused stem: fp32 HWC input -> per-channel int8 quantise (ties-to-even) ->
// conv3x3 s1 p1, 3 -> 64 channels (dp4a over (c0,c1,c2,0) words) -> PReLU epilogue
// -> int8 NHWC, plus the following BN pass as a second output.
// Takes over quantize_fp32_nhwc_to_int8_per_channel + the first conv + its epilogue
// + the first BN (reference kernels/int8_epilogue.c:231-247, kernels/conv2d_nhwc.c:179-220,
// kernels/int8_epilogue.c:25-112 and :253-318) in one pass over the image:
// 150 528 B read and 2 x 802 816 B written per face.
// A block owns a 16x16 output tile: the 18x18 input patch is quantised once into
// shared memory, weights ([tap][co] words) and the per-channel tables sit there too.
// ---------------------------------------------------------------------------
#define STEM_T 16
#define STEM_THREADS 128           // each thread computes two pixels (rows ty and ty + 8 of the tile)
template <bool CONTRACT, bool HAS_SLOPE, bool HAS_BN2, bool CHECK, bool IN_U8>
__global__ void __launch_bounds__(STEM_THREADS) stem_kernel(const void* __restrict__ in_any, const float* __restrict__ inv3,
                                                            const int8_t* __restrict__ w, EpiTables t,
                                                            int8_t* __restrict__ out, int8_t* __restrict__ out2,
                                                            int* __restrict__ q_out)
{
    constexpr int H = 112, W = 112, C = 64, P = STEM_T + 2;
    __shared__ int s_in[P * P];
    __shared__ __align__(16) int s_w[9 * C];          // [tap][co]
    __shared__ __align__(16) float s_tab[4 * C];      // w_scale, bias, slope, inv_out
    __shared__ __align__(16) uint8_t s_lut[HAS_BN2 ? C * 256 : 16];   // the following BN pass as a byte table
    const int b = blockIdx.z;
    const int x0 = blockIdx.x * STEM_T, y0 = blockIdx.y * STEM_T;
    const float i0 = __ldg(inv3), i1 = __ldg(inv3 + 1), i2 = __ldg(inv3 + 2);
    constexpr bool has_bn2 = HAS_BN2;     // compile-time: keeps the per-element code branch-free
    for (int i = threadIdx.x; i < P * P; i += STEM_THREADS) {
        int py = y0 - 1 + i / P, px = x0 - 1 + i % P;
        int v = 0;
        if (py >= 0 && py < H && px >= 0 && px < W) {
            const size_t e = (((size_t)b * H + py) * W + px) * 3;
            float f0, f1, f2;
            if (IN_U8) {
                // 8-bit pixels: the value the reference's wrapper feeds, (p - 127.5) / 127.5 in fp32
                // (fastface.py:11), formed here with the same two roundings
                const uint8_t* x = (const uint8_t*)in_any + e;
                f0 = __fdiv_rn(__fsub_rn((float)__ldg(x), 127.5f), 127.5f);
                f1 = __fdiv_rn(__fsub_rn((float)__ldg(x + 1), 127.5f), 127.5f);
                f2 = __fdiv_rn(__fsub_rn((float)__ldg(x + 2), 127.5f), 127.5f);
            } else {
                const float* x = (const float*)in_any + e;
                f0 = __ldg(x); f1 = __ldg(x + 1); f2 = __ldg(x + 2);
            }
            int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(f0, i0))));
            int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(f1, i1))));
            int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(f2, i2))));
            v = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16);
        }
        s_in[i] = v;
    }
    for (int i = threadIdx.x; i < 9 * C; i += STEM_THREADS) {
        int tap = i / C, co = i % C;
        s_w[i] = __ldg((const int*)w + co * 9 + tap);     // global layout [co][tap] words
    }
    for (int i = threadIdx.x; i < C; i += STEM_THREADS) {
        s_tab[0 * C + i] = t.w_scale[i]; s_tab[1 * C + i] = t.bias[i];
        s_tab[2 * C + i] = t.slope ? t.slope[i] : 0.0f; s_tab[3 * C + i] = t.inv_out[i];
    }
    if (has_bn2)
        for (int i = threadIdx.x; i < C * 16; i += STEM_THREADS) ((int4*)s_lut)[i] = __ldg((const int4*)t.bn_lut + i);
    __syncthreads();
    // Two pixels per thread: every weight word and table entry fetched from shared memory serves
    // both (the kernel is bound by shared-memory reads, two thirds of them weights and tables).
    const int tx = threadIdx.x % STEM_T, ty = threadIdx.x / STEM_T;       // ty in 0..7; second pixel at ty + 8
    int a[2][9];
#pragma unroll
    for (int pp = 0; pp < 2; pp++)
#pragma unroll
        for (int kh = 0; kh < 3; kh++)
#pragma unroll
            for (int kw = 0; kw < 3; kw++) a[pp][kh * 3 + kw] = s_in[(ty + 8 * pp + kh) * P + tx + kw];
    size_t pix[2];
#pragma unroll
    for (int pp = 0; pp < 2; pp++) {
        pix[pp] = ((size_t)b * H + (y0 + ty + 8 * pp)) * W + (x0 + tx);
        if (q_out) q_out[pix[pp]] = a[pp][4];
    }
    constexpr bool has_slope = HAS_SLOPE;
#pragma unroll 1
    for (int g16 = 0; g16 < C / 16; g16++) {          // 16 channels -> one 16-byte store per pixel
        int wo[2][4], wo2[2][4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const int co = g16 * 16 + g * 4;
            int acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
            for (int tap = 0; tap < 9; tap++) {
                const int4 ww = *(const int4*)&s_w[tap * C + co];
#pragma unroll
                for (int pp = 0; pp < 2; pp++) {
                    acc[pp][0] = __dp4a(a[pp][tap], ww.x, acc[pp][0]); acc[pp][1] = __dp4a(a[pp][tap], ww.y, acc[pp][1]);
                    acc[pp][2] = __dp4a(a[pp][tap], ww.z, acc[pp][2]); acc[pp][3] = __dp4a(a[pp][tap], ww.w, acc[pp][3]);
                }
            }
            const float4 ws = *(const float4*)&s_tab[0 * C + co];
            const float4 bi = *(const float4*)&s_tab[1 * C + co];
            const float4 sl = *(const float4*)&s_tab[2 * C + co];
            const float4 iv = *(const float4*)&s_tab[3 * C + co];
#pragma unroll
            for (int pp = 0; pp < 2; pp++) {
                int q0 = ffcu_requant_nosat<CHECK>(ffcu_conv_fp<CONTRACT>(acc[pp][0], ws.x, bi.x, false, 0, 0.0f, has_slope, sl.x), iv.x);
                int q1 = ffcu_requant_nosat<CHECK>(ffcu_conv_fp<CONTRACT>(acc[pp][1], ws.y, bi.y, false, 0, 0.0f, has_slope, sl.y), iv.y);
                int q2 = ffcu_requant_nosat<CHECK>(ffcu_conv_fp<CONTRACT>(acc[pp][2], ws.z, bi.z, false, 0, 0.0f, has_slope, sl.z), iv.z);
                int q3 = ffcu_requant_nosat<CHECK>(ffcu_conv_fp<CONTRACT>(acc[pp][3], ws.w, bi.w, false, 0, 0.0f, has_slope, sl.w), iv.w);
                wo[pp][g] = ffcu_pack4(q0, q1, q2, q3);              // saturates to [-128, 127]
                if (has_bn2) {
                    const uint8_t* lc = s_lut + co * 256;
                    const unsigned w4 = (unsigned)wo[pp][g];
                    const unsigned r0 = lc[w4 & 0xffu], r1 = lc[256 + ((w4 >> 8) & 0xffu)];
                    const unsigned r2 = lc[512 + ((w4 >> 16) & 0xffu)], r3 = lc[768 + (w4 >> 24)];
                    wo2[pp][g] = (int)(r0 | (r1 << 8) | (r2 << 16) | (r3 << 24));
                }
            }
        }
#pragma unroll
        for (int pp = 0; pp < 2; pp++) {
            ((int4*)(out + pix[pp] * C))[g16] = make_int4(wo[pp][0], wo[pp][1], wo[pp][2], wo[pp][3]);
            if (has_bn2) ((int4*)(out2 + pix[pp] * C))[g16] = make_int4(wo2[pp][0], wo2[pp][1], wo2[pp][2], wo2[pp][3]);
        }
    }
}

// Stem weights [co][tap][4] (the dp4a layout) -> [co][32] with k = 3 * tap + c, zero padded.
__global__ void stem_weight_k32_kernel(const int8_t* __restrict__ w, int8_t* __restrict__ wk, int Cout)
{
    const int co = blockIdx.x * blockDim.x + threadIdx.x;
    if (co >= Cout) return;
    for (int k = 0; k < 32; k++) {
        int8_t v = 0;
        if (k < 27) v = w[co * 36 + (k / 3) * 4 + (k % 3)];
        wk[co * 32 + k] = v;
    }
}

int ffcu_stem_weight_k32(const int8_t* d_w, int8_t* d_wk, int Cout, cudaStream_t s)
{
    stem_weight_k32_kernel<<<(Cout + 63) / 64, 64, 0, s>>>(d_w, d_wk, Cout);
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

int ffcu_launch_stem(const void* in_any, int in_u8, const float* inv3, const int8_t* w, const EpiTables& t, int batch,
                     int mode, int8_t* out, int8_t* out_bn2, int8_t* q_out, cudaStream_t s)
{
    dim3 grid(112 / STEM_T, 112 / STEM_T, batch);
    const bool sl = t.slope != nullptr, bn = (out_bn2 != nullptr) && (t.bn_lut != nullptr);
#define STEM_GO(C_, S_, B_) do { \
        if (in_u8) { \
            if (t.no_overflow) stem_kernel<C_, S_, B_, false, true><<<grid, STEM_THREADS, 0, s>>>(in_any, inv3, w, t, out, out_bn2, (int*)q_out); \
            else               stem_kernel<C_, S_, B_, true, true><<<grid, STEM_THREADS, 0, s>>>(in_any, inv3, w, t, out, out_bn2, (int*)q_out); \
        } else { \
            if (t.no_overflow) stem_kernel<C_, S_, B_, false, false><<<grid, STEM_THREADS, 0, s>>>(in_any, inv3, w, t, out, out_bn2, (int*)q_out); \
            else               stem_kernel<C_, S_, B_, true, false><<<grid, STEM_THREADS, 0, s>>>(in_any, inv3, w, t, out, out_bn2, (int*)q_out); \
        } } while (0)
    if (mode) {
        if (sl && bn) STEM_GO(true, true, true); else if (sl) STEM_GO(true, true, false);
        else if (bn) STEM_GO(true, false, true); else STEM_GO(true, false, false);
    } else {
        if (sl && bn) STEM_GO(false, true, true); else if (sl) STEM_GO(false, true, false);
        else if (bn) STEM_GO(false, false, true); else STEM_GO(false, false, false);
    }
#undef STEM_GO
    FFCU_CHECK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// Small-batch FC (batch <= 16): the 12.85 MB weight matrix is the whole cost, so the
// K axis is split across blocks to put every SM on it.  Block (n-group, k-split) computes
// 8 outputs x up to MAXB faces over its K slice with dp4a, reduces across its threads and
// adds the int32 partial sums into a scratch accumulator [batch][N] (integer adds commute,
// so the result is exact).  The block that arrives last at its n-group's ticket counter
// applies out = bias + (float)dot * w_scale (reference kernels/gemm_int8_matvec.c:78-79)
// and leaves sums and ticket at zero for the next call: one launch, no finishing kernel.
//
// The kernel is launched with programmatic stream serialisation: a block requests its weight
// slice (which no kernel writes) BEFORE waiting for the previous kernel, so at batch 1 the
// weight stream is hidden behind the last convolution; the activations are read after the wait.
// MAXB (1, 2, 4, 8, 16 faces) sizes the accumulator registers: at MAXB = 1 all 1 024 blocks are
// resident at once and every weight byte is in flight together.
//
// scratch layout: [FCS_TICKETS] ticket counters, then int32 sums [batch][N]; all zero on entry
// (and again on exit).
// ---------------------------------------------------------------------------
#define FCS_TN 8
#define FCS_MAXB 16
#define FCS_THREADS 128
template <int MAXB, bool CONTRACT>
__global__ void __launch_bounds__(FCS_THREADS) fc_small_kernel(const int8_t* __restrict__ act, const int8_t* __restrict__ w,
                                                               const float* __restrict__ w_scale, const float* __restrict__ bias,
                                                               int B, int N, int K, int k_per_split,
                                                               int* __restrict__ scratch, float* __restrict__ out)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ int red[FCS_THREADS / 32][MAXB * FCS_TN];
    __shared__ int s_last;
    int* tickets = scratch;
    int* sums = scratch + FFCU_FC_SMALL_TICKETS;
    const int n0 = blockIdx.x * FCS_TN;
    const int k0 = blockIdx.y * k_per_split;
    const int kv = k_per_split >> 4;                       // 16-byte steps in this slice
    int acc[MAXB][FCS_TN];
#pragma unroll
    for (int i = 0; i < MAXB; i++)
#pragma unroll
        for (int j = 0; j < FCS_TN; j++) acc[i][j] = 0;
    int k = threadIdx.x;
    int4 ww[FCS_TN];
    if (k < kv) {
#pragma unroll
        for (int j = 0; j < FCS_TN; j++) ww[j] = __ldg((const int4*)(w + (size_t)(n0 + j) * K + k0) + k);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the activations come from the previous kernel
    while (k < kv) {
#pragma unroll
        for (int i = 0; i < MAXB; i++) {
            if (i >= B) break;
            const int4 a = __ldcg((const int4*)(act + (size_t)i * K + k0) + k);
#pragma unroll
            for (int j = 0; j < FCS_TN; j++) {
                int s = acc[i][j];
                s = __dp4a(a.x, ww[j].x, s); s = __dp4a(a.y, ww[j].y, s);
                s = __dp4a(a.z, ww[j].z, s); s = __dp4a(a.w, ww[j].w, s);
                acc[i][j] = s;
            }
        }
        k += FCS_THREADS;
        if (k < kv) {
#pragma unroll
            for (int j = 0; j < FCS_TN; j++) ww[j] = __ldg((const int4*)(w + (size_t)(n0 + j) * K + k0) + k);
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < MAXB; i++) {
        if (i >= B) break;
#pragma unroll
        for (int j = 0; j < FCS_TN; j++) {
            int s = acc[i][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) red[warp][i * FCS_TN + j] = s;
        }
    }
    __syncthreads();
    const int i = threadIdx.x / FCS_TN, j = threadIdx.x % FCS_TN;     // FCS_THREADS = 16 faces x 8 outputs
    if (threadIdx.x < B * FCS_TN) {
        int s = 0;
#pragma unroll
        for (int wv = 0; wv < FCS_THREADS / 32; wv++) s += red[wv][threadIdx.x];
        atomicAdd(sums + (size_t)i * N + n0 + j, s);
        __threadfence();                                   // the partial sum is visible before the ticket is taken
    }
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(tickets + blockIdx.x, 1) == (int)gridDim.y - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();                                       // every other block's sums are visible from here on
    if (threadIdx.x < B * FCS_TN) {
        const int n = n0 + j;
        const int dot = atomicExch(sums + (size_t)i * N + n, 0);      // read and leave clean for the next call
        out[(size_t)i * N + n] = ffcu_fc_fp<CONTRACT>(dot, __ldg(w_scale + n), __ldg(bias + n));
    }
    if (threadIdx.x == 0) tickets[blockIdx.x] = 0;
}

template <int MAXB>
static int fc_small_go(dim3 grid, cudaStream_t s, int mode, const int8_t* act, const int8_t* w, const float* w_scale,
                       const float* bias, int B, int N, int K, int k_per_split, int* scratch, float* out)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(FCS_THREADS);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (mode) FFCU_CHECK(cudaLaunchKernelEx(&cfg, fc_small_kernel<MAXB, true>, act, w, w_scale, bias, B, N, K, k_per_split, scratch, out));
    else      FFCU_CHECK(cudaLaunchKernelEx(&cfg, fc_small_kernel<MAXB, false>, act, w, w_scale, bias, B, N, K, k_per_split, scratch, out));
    return 0;
}

// scratch: FFCU_FC_SMALL_TICKETS + batch * N int32, all zero on entry (and again on exit).
int ffcu_launch_fc_small(const int8_t* act, const int8_t* w, const float* w_scale, const float* bias,
                         int batch, int N, int K, int mode, int* scratch, float* out, cudaStream_t s)
{
    if (batch < 1 || batch > FCS_MAXB || N % FCS_TN != 0 || N / FCS_TN > FFCU_FC_SMALL_TICKETS || K % 16 != 0) {
        ffcu_set_error("small-batch FC needs 1 <= batch <= %d, N %% 8 == 0, N <= %d, K %% 16 == 0", FCS_MAXB,
                       FFCU_FC_SMALL_TICKETS * FCS_TN);
        return -1;
    }
    int splits = 16;
    while (splits > 1 && (K % (splits * 16) != 0)) splits >>= 1;
    const dim3 grid(N / FCS_TN, splits);
    const int kps = K / splits;
    if (batch == 1) return fc_small_go<1>(grid, s, mode, act, w, w_scale, bias, batch, N, K, kps, scratch, out);
    if (batch == 2) return fc_small_go<2>(grid, s, mode, act, w, w_scale, bias, batch, N, K, kps, scratch, out);
    if (batch <= 4) return fc_small_go<4>(grid, s, mode, act, w, w_scale, bias, batch, N, K, kps, scratch, out);
    if (batch <= 8) return fc_small_go<8>(grid, s, mode, act, w, w_scale, bias, batch, N, K, kps, scratch, out);
    return fc_small_go<16>(grid, s, mode, act, w, w_scale, bias, batch, N, K, kps, scratch, out);
}
