/* ref_trace_shim.c -- dump points for the UNMODIFIED reference (TEST INFRASTRUCTURE).
 *
 * Linked next to the reference's own objects with
 *   -Wl,--wrap=fused_epilogue_int8,--wrap=bn_prelu_requant_int8,...
 * so every call the reference driver makes to those kernels lands here first.
 * Each wrapper forwards to the real kernel, then appends one line
 *   <kind> <call#> <n_elems> <crc32-hex>
 * to the file named by $FF_TRACE_OUT (zlib-compatible CRC-32 of the raw bytes).
 *   Q  int8 input after quantisation        (kernels/int8_epilogue.c:218-247)
 *   A  int32 conv accumulators (epilogue input; kernels/int8_epilogue.c:25-112)
 *   O  int8 conv output after the fused epilogue
 *   B  int8 output of a standalone BN pass  (kernels/int8_epilogue.c:253-318)
 *   F  f32 embedding of one face            (kernels/gemm_int8_matvec.c:33-81)
 * With $FF_TRACE_DUMP_DIR set the raw tensors are written there as well.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static FILE* g_out;
static int g_calls[128];

static uint32_t crc32_bytes(const void* data, size_t n)
{
    static uint32_t table[256];
    static int init;
    if (!init) {
        for (uint32_t i = 0; i < 256; i++) {
            uint32_t c = i;
            for (int k = 0; k < 8; k++) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : (c >> 1);
            table[i] = c;
        }
        init = 1;
    }
    const uint8_t* p = (const uint8_t*)data;
    uint32_t c = 0xFFFFFFFFu;
    for (size_t i = 0; i < n; i++) c = table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
    return c ^ 0xFFFFFFFFu;
}

static void record(char kind, const void* data, size_t n_elems, size_t elem_size)
{
    const char* path = getenv("FF_TRACE_OUT");
    if (!path) return;
    if (!g_out) g_out = fopen(path, "w");
    if (!g_out) return;
    int idx = g_calls[(int)kind]++;
    fprintf(g_out, "%c %d %zu %08x\n", kind, idx, n_elems, crc32_bytes(data, n_elems * elem_size));
    fflush(g_out);
    const char* dir = getenv("FF_TRACE_DUMP_DIR");
    if (dir) {
        char name[1024];
        snprintf(name, sizeof name, "%s/%c_%03d.bin", dir, kind, idx);
        FILE* f = fopen(name, "wb");
        if (f) { fwrite(data, elem_size, n_elems, f); fclose(f); }
    }
}

void __real_fused_epilogue_int8(const int32_t* acc, int N_pos, int Cout, float in_scale,
    const float* weight_scales, const float* bias, const float* bn_scale, const float* bn_offset,
    const float* prelu_slope, const int8_t* add_src, float add_scale, const float* add_scale_per_ch,
    const float* inv_out_per_ch, float out_scale, int8_t* out_i8);

void __wrap_fused_epilogue_int8(const int32_t* acc, int N_pos, int Cout, float in_scale,
    const float* weight_scales, const float* bias, const float* bn_scale, const float* bn_offset,
    const float* prelu_slope, const int8_t* add_src, float add_scale, const float* add_scale_per_ch,
    const float* inv_out_per_ch, float out_scale, int8_t* out_i8)
{
    record('A', acc, (size_t)N_pos * Cout, 4);
    __real_fused_epilogue_int8(acc, N_pos, Cout, in_scale, weight_scales, bias, bn_scale, bn_offset,
                               prelu_slope, add_src, add_scale, add_scale_per_ch, inv_out_per_ch,
                               out_scale, out_i8);
    record('O', out_i8, (size_t)N_pos * Cout, 1);
}

void __real_bn_prelu_requant_int8(const int8_t* in_i8, float in_scale, const float* in_scale_per_ch,
    const float* bn_scale, const float* bn_offset, const float* prelu_slope,
    const float* inv_out_per_ch, float out_scale, int8_t* out_i8, int N_pos, int C);

void __wrap_bn_prelu_requant_int8(const int8_t* in_i8, float in_scale, const float* in_scale_per_ch,
    const float* bn_scale, const float* bn_offset, const float* prelu_slope,
    const float* inv_out_per_ch, float out_scale, int8_t* out_i8, int N_pos, int C)
{
    __real_bn_prelu_requant_int8(in_i8, in_scale, in_scale_per_ch, bn_scale, bn_offset, prelu_slope,
                                 inv_out_per_ch, out_scale, out_i8, N_pos, C);
    record('B', out_i8, (size_t)N_pos * C, 1);
}

void __real_fastface_gemm_i8_matvec_vnni(const uint8_t* Au, const int8_t* W, const int32_t* w_row_sum,
    const float* W_scale, const float* bias, float A_scale, float* out, int N, int K);

void __wrap_fastface_gemm_i8_matvec_vnni(const uint8_t* Au, const int8_t* W, const int32_t* w_row_sum,
    const float* W_scale, const float* bias, float A_scale, float* out, int N, int K)
{
    __real_fastface_gemm_i8_matvec_vnni(Au, W, w_row_sum, W_scale, bias, A_scale, out, N, K);
    record('F', out, (size_t)N, 4);
}

void __real_quantize_fp32_nhwc_to_int8_per_channel(const float* in, int N_pos, int C,
    const float* inv_scale_per_ch, int8_t* out);

void __wrap_quantize_fp32_nhwc_to_int8_per_channel(const float* in, int N_pos, int C,
    const float* inv_scale_per_ch, int8_t* out)
{
    __real_quantize_fp32_nhwc_to_int8_per_channel(in, N_pos, C, inv_scale_per_ch, out);
    record('Q', out, (size_t)N_pos * C, 1);
}

void __real_quantize_fp32_nhwc_to_int8(const float* in, int N, float scale, int8_t* out);

void __wrap_quantize_fp32_nhwc_to_int8(const float* in, int N, float scale, int8_t* out)
{
    __real_quantize_fp32_nhwc_to_int8(in, N, scale, out);
    record('Q', out, (size_t)N, 1);
}
