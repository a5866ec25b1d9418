// ffcu_context.cu -- device context behind include/ff_cuda.h: buffers, the static
// launch list, submit / wait, dump points and the resident-input timing loop.

#include "ffcu_internal.cuh"
#include <math.h>

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <map>
#include <vector>

static thread_local char g_cu_err[512];

void ffcu_set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_cu_err, sizeof g_cu_err, fmt, ap);
    va_end(ap);
}

extern "C" const char* ffcu_last_error(void) { return g_cu_err; }

struct DevLayer {
    ffcu_layer d;          // host-side description; pointer members are NOT valid on the device
    int8_t* w = nullptr;
    float* tab[12] = {};   // w_scale,bias,slope,res_scale,inv_out | in_scale,bn_scale,bn_offset | bn2 in,scale,offset,inv
    EpiTables epi{};
    TcPlan* tc = nullptr;  // non-NULL: tensor-core implicit GEMM takes this layer (plan with the widest column tile)
    TcPlan* tc_bn[3] = {}; // plans for column tiles of 64 / 128 / 256 channels, made when a call first needs them
    int8_t* bn_lut = nullptr;  // device copy of the fused BN's table
    bool fused_stem = false;   // conv that also does the input quantisation (reads the fp32 input)
    bool skip = false;         // quantise layer absorbed by the fused stem
    StemTcPlan* stem_tc = nullptr; // fused stem on tensor cores, one launch (else the dp4a stem kernel)
    ScPlan* sc = nullptr;          // this stride-2 conv and the next layer (the block's 1x1 shortcut) as one launch
    int sc_write_main = 0;         // ... which must still store this layer's output: a later layer reads it
    int8_t* wk32 = nullptr;        // its weights repacked [64][32]
};

struct ffcu_ctx {
    int device = 0;
    int max_batch = 0;
    int n_bufs = 0;
    size_t bytes_per_face = 0;
    int8_t* bufs[FFCU_MAX_BUFS] = {};
    // Two input / output slots: the H2D copy of step k+1 and the D2H copy of step k-1
    // overlap the kernels of step k (copy-in, compute and copy-out streams).
    float* in_slot[2] = {};      // [max_batch][112][112][3] f32
    float* out_slot[2] = {};     // [max_batch][512] f32
    float* d_in = nullptr;       // slot the next launch_forward reads
    bool in_u8 = false;          // that slot holds 8-bit pixels [n][112][112][3] instead of fp32
    float* d_out = nullptr;      // slot the next launch_forward writes
    cudaEvent_t ev_in_ready[2] = {}, ev_compute_done[2] = {}, ev_out_copied[2] = {};
    unsigned long long seq = 0;
    int* d_fc_scratch = nullptr; // small-batch FC: 64 ticket counters + int32 [16][512] split-K accumulator (kept zero between calls)
    int* d_err = nullptr;        // device error word
    int* h_err = nullptr;        // pinned mirror
    cudaStream_t stream = nullptr;       // compute
    cudaStream_t s_in = nullptr, s_out = nullptr;
    std::vector<DevLayer> layers;
    int mode = 1;
    int force_simt = 0;          // FF_CONV_IMPL=simt: every conv on the CUDA-core kernel
    int no_fc_small = 0;         // FF_FC_SMALL=0: small batches take the large-batch FC path too
    int fc_small_max = 4;        // largest batch the CUDA-core FC kernel takes ($FF_FC_SMALL_MAX, at most 16): measured quicker than the split-K tensor-core FC up to 3 faces, equal at 4, slower from 6
    int* d_fc_tc_scratch = nullptr; // split-K tensor-core FC: FFCU_FC_TC_TICKETS counters + int32 [fc_tc_rows][512] sums (kept zero between calls)
    int fc_tc_rows = 0;
    int launches = 0;
    bool finalized = false;
    // The forward is captured once per (batch, mode, input kind, input/output slot) into a CUDA
    // graph and replayed: small batches are launch-bound (55 short kernels), large ones still
    // save the host's launch work.  FF_GRAPH=0 disables (0), FF_GRAPH_MAX_BATCH caps the batch.
    int graph_max_batch = 1 << 30;
    std::map<long long, cudaGraphExec_t> graphs;
    std::map<long long, int> graph_launches;
    // Batch 1: runs of same-shape 3x3 stride-1 convolutions (the 14x14 and 7x7 stages) go out as one
    // launch each (conv_tc_chain.cu).  Found on the first one-face forward; FF_CHAIN=0 disables.
    // Calls of at most lean_max_batch faces run copy-in, forward and copy-out on the compute stream alone
    // (FF_LEAN_MAX_BATCH, default 1: the single-face call; 0 = always the three-stream pipeline, whose overlap of
    // the next call's copy-in with this call's kernels is worth more than the hops it costs from a few faces up).
    int lean_max_batch = 1;
    bool lean_last = false;      // the previous submit took that path
    bool err_copied = false;     // ... and queued the error word's copy already
    struct Chain { size_t first; int count; ChainPlan* plan; };
    std::vector<Chain> chains;
    bool chains_built = false;
    int no_chain = 0;
};

extern "C" int ffcu_device_count(void)
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { ffcu_set_error("cudaGetDeviceCount: %s", cudaGetErrorString(e)); return -1; }
    return n;
}

static float* upload_f32(const float* src, int n)
{
    if (!src) return nullptr;
    float* d = nullptr;
    if (cudaMalloc(&d, (size_t)n * sizeof(float)) != cudaSuccess) return nullptr;
    if (cudaMemcpy(d, src, (size_t)n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(d); return nullptr; }
    return d;
}

extern "C" ffcu_ctx* ffcu_create(int device, int max_batch, int n_bufs, size_t bytes_per_face)
{
    if (n_bufs < 1 || n_bufs > FFCU_MAX_BUFS || max_batch < 1) { ffcu_set_error("bad ffcu_create arguments"); return nullptr; }
    if (cudaSetDevice(device) != cudaSuccess) { ffcu_set_error("cudaSetDevice(%d) failed", device); return nullptr; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { ffcu_set_error("cudaGetDeviceProperties failed"); return nullptr; }
    if (prop.major != 10) {
        ffcu_set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return nullptr;
    }
    ffcu_ctx* c = new ffcu_ctx();
    c->device = device; c->max_batch = max_batch; c->n_bufs = n_bufs; c->bytes_per_face = bytes_per_face;
    bool ok = true;
    // 1 KiB of slack after each tensor: TMA boxes of partial tiles stay inside the allocation
    size_t act = (size_t)max_batch * bytes_per_face + 1024;
    for (int i = 0; i < n_bufs && ok; i++) ok = cudaMalloc(&c->bufs[i], act) == cudaSuccess;
    for (int k = 0; k < 2; k++) {
        ok = ok && cudaMalloc(&c->in_slot[k], (size_t)max_batch * 37632 * sizeof(float)) == cudaSuccess;
        ok = ok && cudaMalloc(&c->out_slot[k], (size_t)max_batch * 512 * sizeof(float)) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&c->ev_in_ready[k], cudaEventDisableTiming) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&c->ev_compute_done[k], cudaEventDisableTiming) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&c->ev_out_copied[k], cudaEventDisableTiming) == cudaSuccess;
    }
    c->d_in = c->in_slot[0]; c->d_out = c->out_slot[0];
    ok = ok && cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaMalloc(&c->d_err, sizeof(int)) == cudaSuccess;
    ok = ok && cudaMalloc(&c->d_fc_scratch, (FFCU_FC_SMALL_TICKETS + FFCU_FC_SMALL_MAX_BATCH * 512) * sizeof(int)) == cudaSuccess;
    if (ok) cudaMemset(c->d_fc_scratch, 0, (FFCU_FC_SMALL_TICKETS + FFCU_FC_SMALL_MAX_BATCH * 512) * sizeof(int));
    c->fc_tc_rows = (max_batch + 127) / 128 * 128;
    {
        const size_t nb = ((size_t)FFCU_FC_TC_TICKETS + (size_t)c->fc_tc_rows * 512) * sizeof(int);
        ok = ok && cudaMalloc(&c->d_fc_tc_scratch, nb) == cudaSuccess;
        if (ok) cudaMemset(c->d_fc_tc_scratch, 0, nb);
    }
    ok = ok && cudaHostAlloc(&c->h_err, sizeof(int), cudaHostAllocDefault) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) == cudaSuccess;
    if (ok) { cudaMemset(c->d_err, 0, sizeof(int)); *c->h_err = 0; }
    const char* impl = getenv("FF_CONV_IMPL");
    c->force_simt = (impl && strcmp(impl, "simt") == 0) ? 1 : 0;
    { const char* e = getenv("FF_FC_SMALL"); c->no_fc_small = (e && e[0] == '0') ? 1 : 0; }
    { const char* e = getenv("FF_FC_SMALL_MAX"); if (e && atoi(e) >= 0 && atoi(e) <= FFCU_FC_SMALL_MAX_BATCH) c->fc_small_max = atoi(e); }
    { const char* e = getenv("FF_GRAPH_MAX_BATCH"); if (e && atoi(e) > 0) c->graph_max_batch = atoi(e); }
    { const char* e = getenv("FF_GRAPH"); if (e && e[0] == '0') c->graph_max_batch = 0; }
    { const char* e = getenv("FF_CHAIN"); c->no_chain = (e && e[0] == '0') ? 1 : 0; }
    { const char* e = getenv("FF_LEAN_MAX_BATCH"); if (e && atoi(e) >= 0) c->lean_max_batch = atoi(e); }
    if (!ok) {
        ffcu_set_error("device allocation failed on device %d: %s", device, cudaGetErrorString(cudaGetLastError()));
        ffcu_destroy(c);
        return nullptr;
    }
    return c;
}

static void free_layer_memory(DevLayer& L);

extern "C" void ffcu_destroy(ffcu_ctx* c)
{
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->s_in) cudaStreamSynchronize(c->s_in);
    if (c->s_out) cudaStreamSynchronize(c->s_out);
    for (auto& g : c->graphs) cudaGraphExecDestroy(g.second);
    for (auto& ch : c->chains) ffcu_chain_free(ch.plan);
    for (auto& L : c->layers) {
        for (TcPlan* q : L.tc_bn) if (q) ffcu_tc_free(q);      // L.tc is one of them
        if (L.stem_tc) ffcu_stem_tc_free(L.stem_tc);
        if (L.sc) ffcu_sc_free(L.sc);
        free_layer_memory(L);
    }
    for (int i = 0; i < FFCU_MAX_BUFS; i++) cudaFree(c->bufs[i]);
    for (int k = 0; k < 2; k++) {
        cudaFree(c->in_slot[k]); cudaFree(c->out_slot[k]);
        if (c->ev_in_ready[k]) cudaEventDestroy(c->ev_in_ready[k]);
        if (c->ev_compute_done[k]) cudaEventDestroy(c->ev_compute_done[k]);
        if (c->ev_out_copied[k]) cudaEventDestroy(c->ev_out_copied[k]);
    }
    cudaFree(c->d_err); cudaFree(c->d_fc_scratch); cudaFree(c->d_fc_tc_scratch);
    if (c->h_err) cudaFreeHost(c->h_err);
    if (c->stream) cudaStreamDestroy(c->stream);
    if (c->s_in) cudaStreamDestroy(c->s_in);
    if (c->s_out) cudaStreamDestroy(c->s_out);
    delete c;
}

// True when no int8 input can drive the requantised value of this conv layer near the range
// of a 32-bit integer: |acc| <= 128 * sum|w|, so per channel
//   |t| <= (128 * sum|w| * |w_scale| + |bias| + 128 * |res_scale|) * max(1, |slope|)
// and the converted value is at most |t| * |inv_out| + 0.5.  The bound is evaluated in double
// and compared with 2^30, a factor two inside the limit to cover the fp32 roundings.
static bool epilogue_cannot_overflow(const ffcu_layer* l)
{
    if (l->kind != FFCU_CONV || !l->w || !l->w_scale || !l->bias || !l->inv_out || l->Cout < 1) return false;
    const size_t K = l->w_bytes / (size_t)l->Cout;
    for (int c = 0; c < l->Cout; c++) {
        double s = 0.0;
        const int8_t* wr = l->w + (size_t)c * K;
        for (size_t k = 0; k < K; k++) s += fabs((double)wr[k]);
        double t = 128.0 * s * fabs((double)l->w_scale[c]) + fabs((double)l->bias[c]);
        if (l->res_scale) t += 128.0 * fabs((double)l->res_scale[c]);
        if (l->slope) { const double a = fabs((double)l->slope[c]); if (a > 1.0) t *= a; if (!(a == a)) return false; }
        const double q = t * fabs((double)l->inv_out[c]) + 1.0;
        if (!(q < 1073741824.0)) return false;            // also rejects NaN / inf
        if (l->bn2_in_scale && l->bn2_scale && l->bn2_offset && l->bn2_inv_out) {
            // the fused BN of the int8 result: |128 * in_scale * scale + offset| * inv_out
            const double b = (128.0 * fabs((double)l->bn2_in_scale[c]) * fabs((double)l->bn2_scale[c]) +
                              fabs((double)l->bn2_offset[c])) * fabs((double)l->bn2_inv_out[c]) + 1.0;
            if (!(b < 1073741824.0)) return false;
        }
    }
    return true;
}

// True when |accumulator| <= 128 * sum|w| stays below 2^22 for every output channel of this conv layer.
static bool accumulator_fits_22_bits(const ffcu_layer* l)
{
    if (l->kind != FFCU_CONV || !l->w || l->Cout < 1) return false;
    const size_t K = l->w_bytes / (size_t)l->Cout;
    for (int c = 0; c < l->Cout; c++) {
        long long s = 0;
        const int8_t* wr = l->w + (size_t)c * K;
        for (size_t k = 0; k < K; k++) s += wr[k] < 0 ? -(long long)wr[k] : (long long)wr[k];
        if (128 * s >= (1ll << 22)) return false;
    }
    return true;
}

static void free_layer_memory(DevLayer& L)
{
    cudaFree(L.w); L.w = nullptr;
    cudaFree(L.bn_lut); L.bn_lut = nullptr;
    for (float*& t : L.tab) { cudaFree(t); t = nullptr; }
    cudaFree(L.wk32); L.wk32 = nullptr;
}

extern "C" int ffcu_add_layer(ffcu_ctx* c, const ffcu_layer* l)
{
    if (!c || !l || c->finalized) { ffcu_set_error("ffcu_add_layer: bad state"); return -1; }
    cudaSetDevice(c->device);
    DevLayer L;
    L.d = *l;
    const int C = l->Cout;
    // every early return below goes through fail(): nothing uploaded for this layer stays allocated
    auto fail = [&](const char* what) { ffcu_set_error("%s", what); free_layer_memory(L); cudaGetLastError(); return -1; };
    if (l->bn2_dst_buf >= 0 && !(l->bn2_in_scale && l->bn2_scale && l->bn2_offset && l->bn2_inv_out))
        return fail("fused BN output without its tables");
    if (l->w && l->w_bytes) {
        if (cudaMalloc(&L.w, l->w_bytes + 1024) != cudaSuccess) return fail("weight allocation failed");
        if (cudaMemset(L.w, 0, l->w_bytes + 1024) != cudaSuccess ||
            cudaMemcpy(L.w, l->w, l->w_bytes, cudaMemcpyHostToDevice) != cudaSuccess) return fail("weight upload failed");
    }
    const float* src[12] = {l->w_scale, l->bias, l->slope, l->res_scale, l->inv_out, l->in_scale, l->bn_scale, l->bn_offset,
                            l->bn2_in_scale, l->bn2_scale, l->bn2_offset, l->bn2_inv_out};
    for (int k = 0; k < 12; k++) {
        int n = (l->kind == FFCU_QUANT) ? 3 : C;
        if (src[k]) {
            L.tab[k] = upload_f32(src[k], n);
            if (!L.tab[k]) return fail("table allocation or upload failed");
        }
    }
    L.epi.w_scale = L.tab[0]; L.epi.bias = L.tab[1]; L.epi.slope = L.tab[2];
    L.epi.res_scale = L.tab[3]; L.epi.inv_out = L.tab[4];
    L.epi.bn_in = L.tab[8]; L.epi.bn_scale = L.tab[9]; L.epi.bn_offset = L.tab[10]; L.epi.bn_inv = L.tab[11];
    if (l->bn2_dst_buf >= 0) {
        std::vector<int8_t> lut((size_t)C * 256);
        if (l->bn2_lut) memcpy(lut.data(), l->bn2_lut, lut.size());
        else ff_bn_lut_build(l->bn2_in_scale, l->bn2_scale, l->bn2_offset, l->bn2_inv_out, C, lut.data());
        if (cudaMalloc(&L.bn_lut, lut.size()) != cudaSuccess) return fail("BN table allocation failed");
        if (cudaMemcpy(L.bn_lut, lut.data(), lut.size(), cudaMemcpyHostToDevice) != cudaSuccess) return fail("BN table upload failed");
    }
    L.epi.bn_lut = L.bn_lut;
    L.epi.no_overflow = epilogue_cannot_overflow(l) ? 1 : 0;
    L.epi.acc22 = accumulator_fits_22_bits(l) ? 1 : 0;
    L.d.bn2_lut = nullptr;
    L.d.bn2_in_scale = L.d.bn2_scale = L.d.bn2_offset = L.d.bn2_inv_out = nullptr;
    L.d.w = nullptr;
    L.d.w_scale = L.d.bias = L.d.slope = L.d.res_scale = L.d.inv_out = nullptr;
    L.d.in_scale = L.d.bn_scale = L.d.bn_offset = nullptr;
    if (cudaGetLastError() != cudaSuccess) return fail("upload failed");
    c->layers.push_back(L);
    return (int)c->layers.size() - 1;
}

extern "C" int ffcu_finalize(ffcu_ctx* c)
{
    if (!c) return -1;
    cudaSetDevice(c->device);
    for (auto& L : c->layers) {
        if ((L.d.kind == FFCU_CONV || L.d.kind == FFCU_FC) && !c->force_simt) {
            if (L.d.src_buf < 0 || L.d.src_buf >= c->n_bufs) { ffcu_set_error("layer source buffer out of range"); return -1; }
            const int bn = L.d.Cout >= 256 ? 256 : L.d.Cout;
            L.tc = ffcu_tc_plan(L.d, c->max_batch, c->bufs[L.d.src_buf], L.w, c->device, bn);
            if (L.tc) L.tc_bn[bn == 64 ? 0 : bn == 128 ? 1 : 2] = L.tc;
        }
    }
    // [quantise, conv3x3 3->64 s1 p1 at 112x112] -> one fused stem kernel
    const char* fs = getenv("FF_FUSE_STEM");
    if (!c->force_simt && !(fs && fs[0] == '0') && c->layers.size() >= 2) {
        DevLayer& q = c->layers[0]; DevLayer& s = c->layers[1];
        if (q.d.kind == FFCU_QUANT && s.d.kind == FFCU_CONV && !s.tc && s.d.src_buf == q.d.dst_buf && s.d.Cin == 3 &&
            s.d.Cin_pad == 4 && s.d.Cout == 64 && s.d.Kh == 3 && s.d.Kw == 3 && s.d.stride == 1 && s.d.pad == 1 &&
            s.d.H == 112 && s.d.W == 112 && s.d.res_buf < 0) {
            s.fused_stem = true; q.skip = true;
            // tensor-core form: im2col rows built in shared memory, K = 32 GEMM, all in one launch
            const char* st = getenv("FF_STEM_TC");
            if (!(st && st[0] == '0') && s.epi.no_overflow && s.epi.slope) {
                if (cudaMalloc(&s.wk32, 64 * 32) == cudaSuccess &&
                    ffcu_stem_weight_k32(s.w, s.wk32, 64, c->stream) == 0 && cudaStreamSynchronize(c->stream) == cudaSuccess)
                    s.stem_tc = ffcu_stem_tc_plan(c->max_batch, s.wk32, s.d.bn2_dst_buf >= 0, c->device);
                if (!s.stem_tc) { cudaFree(s.wk32); s.wk32 = nullptr; cudaGetLastError(); }
            }
        }
    }
    // [conv 3x3 stride 2] -> [conv 1x1 stride 2 on the block's input, ADD of the former's output fused]: one launch
    // where the call's column tile is 64 channels wide (conv_tc_sc.cu).  FF_FUSE_SC=0 keeps the two launches.
    const char* fsc = getenv("FF_FUSE_SC");
    if (!c->force_simt && !(fsc && fsc[0] == '0')) {
        for (size_t k = 0; k + 1 < c->layers.size(); k++) {
            DevLayer& M = c->layers[k]; DevLayer& S = c->layers[k + 1];
            const ffcu_layer& m = M.d; const ffcu_layer& sd = S.d;
            if (m.kind != FFCU_CONV || sd.kind != FFCU_CONV || !M.tc || !S.tc || M.fused_stem) continue;
            if (m.stride != 2 || m.Kh != 3 || m.res_buf >= 0 || m.bn2_dst_buf >= 0 || sd.Kh != 1 || sd.stride != 2) continue;
            if (sd.res_buf != m.dst_buf || sd.res_buf < 0 || !S.epi.res_scale) continue;
            if (!M.epi.no_overflow || !S.epi.no_overflow) continue;
            if (sd.bn2_dst_buf >= 0 && !S.bn_lut) continue;
            if (sd.src_buf < 0 || sd.src_buf >= c->n_bufs) continue;
            // One launch reads both layers' inputs while it writes the shortcut's outputs (and, tile by tile, long after
            // other tiles' outputs are out): an output that shares a buffer with an input would overwrite pixels other
            // CTAs have yet to read.  As two launches that sharing is legal (the 3x3 conv's input is dead by then).
            if (sd.dst_buf == m.src_buf || sd.dst_buf == sd.src_buf || m.dst_buf == m.src_buf || m.dst_buf == sd.src_buf ||
                (sd.bn2_dst_buf >= 0 && (sd.bn2_dst_buf == m.src_buf || sd.bn2_dst_buf == sd.src_buf))) continue;
            // does anything after the shortcut still read the main path's tensor before it is overwritten?
            int write_main = 0;
            for (size_t j = k + 2; j < c->layers.size(); j++) {
                const ffcu_layer& o = c->layers[j].d;
                if (o.src_buf == m.dst_buf || o.res_buf == m.dst_buf) { write_main = 1; break; }
                if (o.dst_buf == m.dst_buf || o.bn2_dst_buf == m.dst_buf) break;
            }
            M.sc = ffcu_sc_plan(m, sd, c->max_batch, c->bufs[m.src_buf], M.w, c->bufs[sd.src_buf], S.w, c->device);
            M.sc_write_main = write_main;
        }
    }
    c->launches = 0;
    for (auto& L : c->layers) if (!L.skip) c->launches++;
    c->finalized = true;
    return 0;
}

extern "C" int ffcu_set_mode(ffcu_ctx* c, int mode)
{
    if (!c || (mode != 0 && mode != 1)) return -1;
    c->mode = mode;
    return 0;
}

extern "C" int ffcu_launches_per_forward(const ffcu_ctx* c) { return c ? c->launches : 0; }

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------

// The layer's plan for a call of n faces: the column tile follows the batch of the CALL (one face
// through a context made for 256 gets the narrow tiles that spread a layer over the SMs), so the
// reference's create + embed sequence needs no hint about the batch it will see.
static TcPlan* tc_plan_for(ffcu_ctx* c, DevLayer& L, int n)
{
    if (!L.tc) return nullptr;
    const int bn = ffcu_tc_pick_bn(L.d, n, c->device);
    const int slot = bn == 64 ? 0 : bn == 128 ? 1 : 2;
    if (!L.tc_bn[slot]) {
        L.tc_bn[slot] = ffcu_tc_plan(L.d, c->max_batch, c->bufs[L.d.src_buf], L.w, c->device, bn);
        if (!L.tc_bn[slot]) return L.tc;
    }
    return L.tc_bn[slot];
}

// Launch layer k for n faces.  acc_dbg (optional) receives the conv's int32 accumulators;
// unfused = dump-point mode: the stem runs as separate quantise + conv launches.
static int launch_layer(ffcu_ctx* c, size_t k, int n, int32_t* acc_dbg, bool unfused = false)
{
    DevLayer& L = c->layers[k];
    const ffcu_layer& d = L.d;
    cudaStream_t s = c->stream;
    int8_t* out2 = d.bn2_dst_buf >= 0 ? c->bufs[d.bn2_dst_buf] : nullptr;
    switch (d.kind) {
    case FFCU_QUANT:
        if (L.skip && !unfused) return 0;
        if (c->in_u8) { ffcu_set_error("8-bit pixel input needs the fused stem (FF_FUSE_STEM=0 or a dump-point run is in effect)"); return -1; }
        return ffcu_launch_quant(c->d_in, n * d.H * d.W, L.tab[4], c->bufs[d.dst_buf], s);
    case FFCU_CONV: {
        const int8_t* res = d.res_buf >= 0 ? c->bufs[d.res_buf] : nullptr;
        if (L.fused_stem && !unfused && L.stem_tc)
            return ffcu_stem_fused_launch(L.stem_tc, c->d_in, c->in_u8 ? 1 : 0, c->layers[0].tab[4], n, c->mode, L.epi,
                                          c->bufs[d.dst_buf], out2, c->d_err, s);
        if (L.fused_stem && !unfused)
            return ffcu_launch_stem(c->d_in, c->in_u8 ? 1 : 0, c->layers[0].tab[4], L.w, L.epi, n, c->mode, c->bufs[d.dst_buf], out2, nullptr, s);
        if (L.tc) return ffcu_tc_launch(tc_plan_for(c, L, n), n, c->mode, L.epi, res, acc_dbg, c->bufs[d.dst_buf], out2, c->d_err, s);
        return ffcu_launch_conv_simt(d, n, c->mode, c->bufs[d.src_buf], L.w, L.epi, res, acc_dbg, c->bufs[d.dst_buf], out2, s);
    }
    case FFCU_BN:
        return ffcu_launch_bn(c->bufs[d.src_buf], c->bufs[d.dst_buf], (size_t)n * d.H * d.W, d.Cout,
                              L.tab[5], L.tab[6], L.tab[7], L.tab[4], s);
    case FFCU_FC:
        if (n <= c->fc_small_max && d.Cout <= 512 && !c->no_fc_small)
            return ffcu_launch_fc_small(c->bufs[d.src_buf], L.w, L.epi.w_scale, L.epi.bias, n, d.Cout, d.Cin, c->mode,
                                        c->d_fc_scratch, c->d_out, s);
        if (L.tc) {
            TcPlan* fp = tc_plan_for(c, L, n);
            const int rc = d.Cout == 512 ? ffcu_fc_tc_launch(fp, n, c->mode, L.epi, c->d_out, c->d_fc_tc_scratch, c->fc_tc_rows, c->d_err, s) : 1;
            if (rc <= 0) return rc;
            return ffcu_tc_launch(fp, n, c->mode, L.epi, nullptr, nullptr, c->d_out, nullptr, c->d_err, s);
        }
        return ffcu_launch_fc_simt(c->bufs[d.src_buf], L.w, L.epi.w_scale, L.epi.bias, n, d.Cout, d.Cin,
                                   c->mode, c->d_out, s);
    }
    ffcu_set_error("unknown layer kind %d", d.kind);
    return -1;
}

// A layer the chain kernel can take: tensor-core 3x3 stride-1 pad-1 convolution C -> C (C = 256 or 512)
// with the no-overflow proof, its fused BN (if any) as a byte table.
static bool chain_eligible(const ffcu_ctx* c, const DevLayer& L)
{
    const ffcu_layer& d = L.d;
    return d.kind == FFCU_CONV && L.tc && !L.skip && !L.fused_stem && !c->force_simt && d.Kh == 3 && d.Kw == 3 &&
           d.stride == 1 && d.pad == 1 && d.Cin_pad == d.Cout && d.Cin == d.Cout && d.Cout % 128 == 0 && d.H == d.W &&
           d.Ho == d.H && d.Wo == d.W && L.epi.no_overflow && (d.bn2_dst_buf < 0 || L.bn_lut != nullptr);
}

static void build_chains(ffcu_ctx* c)
{
    c->chains_built = true;
    if (c->no_chain) return;
    size_t k = 0;
    while (k < c->layers.size()) {
        if (!chain_eligible(c, c->layers[k])) { k++; continue; }
        size_t e = k + 1;
        while (e < c->layers.size() && chain_eligible(c, c->layers[e]) && c->layers[e].d.H == c->layers[k].d.H &&
               c->layers[e].d.Cout == c->layers[k].d.Cout) {
            const ffcu_layer& prev = c->layers[e - 1].d;
            const int feeds = prev.bn2_dst_buf >= 0 ? prev.bn2_dst_buf : prev.dst_buf;
            if (c->layers[e].d.src_buf != feeds) break;
            e++;
        }
        const int count = (int)(e - k);
        if (count >= 2) {
            std::vector<ChainLayerDesc> desc((size_t)count);
            for (int i = 0; i < count; i++) {
                const DevLayer& L = c->layers[k + i];
                desc[i].w = L.w; desc[i].t = L.epi;
                desc[i].res = L.d.res_buf >= 0 ? c->bufs[L.d.res_buf] : nullptr;
                desc[i].out = c->bufs[L.d.dst_buf];
                desc[i].out2 = L.d.bn2_dst_buf >= 0 ? c->bufs[L.d.bn2_dst_buf] : nullptr;
            }
            const ffcu_layer& d0 = c->layers[k].d;
            ChainPlan* plan = ffcu_chain_plan(d0.H, d0.W, d0.Cout, c->bufs[d0.src_buf], desc.data(), count, c->device);
            if (plan) c->chains.push_back({k, count, plan});
        }
        k = e;
    }
}

static int launch_forward(ffcu_ctx* c, int n)
{
    int launches = 0;
    if (n == 1 && !c->chains_built) build_chains(c);
    size_t next_chain = 0;
    for (size_t k = 0; k < c->layers.size(); k++) {
        if (n == 1) {
            while (next_chain < c->chains.size() && c->chains[next_chain].first < k) next_chain++;
            if (next_chain < c->chains.size() && c->chains[next_chain].first == k) {
                const ffcu_ctx::Chain& ch = c->chains[next_chain];
                if (ffcu_chain_launch(ch.plan, c->mode, c->d_err, c->stream) == 0) {
                    launches++;
                    k += (size_t)ch.count - 1;
                    continue;
                }
                // the cluster launch was refused (no eight free SMs in one GPC right now, a partitioned device ...):
                // drop the chains for this context and go on with this layer as a launch of its own
                cudaGetLastError();
                for (auto& gone : c->chains) ffcu_chain_free(gone.plan);
                c->chains.clear();
                c->no_chain = 1;
            }
        }
        {
            DevLayer& M = c->layers[k];
            if (M.sc && ffcu_tc_pick_bn(M.d, n, c->device, 1) == 64) {
                // stride-2 conv + the block's shortcut, one launch
                DevLayer& S = c->layers[k + 1];
                int8_t* out2 = S.d.bn2_dst_buf >= 0 ? c->bufs[S.d.bn2_dst_buf] : nullptr;
                int rc = ffcu_sc_launch(M.sc, n, c->mode, M.epi, S.epi, c->bufs[M.d.dst_buf], M.sc_write_main,
                                        c->bufs[S.d.dst_buf], out2, c->d_err, c->stream);
                if (rc != 0) return rc;
                launches++;
                k++;
                continue;
            }
        }
        int rc = launch_layer(c, k, n, nullptr);
        if (rc != 0) return rc;
        const DevLayer& L = c->layers[k];
        if (!L.skip) launches++;
    }
    c->launches = launches;
    return 0;
}

// Forward for n faces on the compute stream: replay of a captured graph for small batches
// (after one eager run of that shape, which also sets the kernels' one-time attributes).
static int run_forward(ffcu_ctx* c, int n, int slot)
{
    if (n > c->graph_max_batch) return launch_forward(c, n);
    const long long key = ((long long)n << 8) | ((long long)c->mode << 4) | (c->in_u8 ? 2 : 0) | slot;
    auto it = c->graphs.find(key);
    if (it != c->graphs.end()) {
        FFCU_CHECK(cudaGraphLaunch(it->second, c->stream));
        c->launches = c->graph_launches[key];
        return 0;
    }
    auto seen = c->graph_launches.find(key);
    if (seen == c->graph_launches.end()) {          // first time: eager
        int rc = launch_forward(c, n);
        if (rc == 0) c->graph_launches[key] = c->launches;
        return rc;
    }
    if (c->graphs.size() >= 64) return launch_forward(c, n);   // a serving loop with many distinct batch sizes: stay eager beyond 64 graphs
    cudaGraph_t graph = nullptr;
    FFCU_CHECK(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    int rc = launch_forward(c, n);
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    if (rc != 0 || e != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        c->graph_max_batch = 0;                     // capture not possible here: stay eager
        return rc != 0 ? rc : launch_forward(c, n);
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess || !exec) { cudaGetLastError(); c->graph_max_batch = 0; return launch_forward(c, n); }
    c->graphs[key] = exec;
    FFCU_CHECK(cudaGraphLaunch(exec, c->stream));
    return 0;
}

static int submit_impl(ffcu_ctx* c, const void* host_in, size_t bytes_per_face, bool u8, int n, float* host_out)
{
    if (!c || !c->finalized || !host_in || !host_out || n < 1 || n > c->max_batch) {
        ffcu_set_error("ffcu_submit: bad arguments");
        return -1;
    }
    FFCU_CHECK(cudaSetDevice(c->device));
    const int slot = (int)(c->seq & 1);
    const bool reused = c->seq >= 2;
    if (n <= c->lean_max_batch) {
        // Latency path (a handful of faces): copy-in, forward and copy-out in order on the compute stream.  The three-
        // stream pipeline below buys overlap a small batch has no use for and costs it two cross-stream hops and a
        // dozen driver calls per face.
        if (!c->lean_last) {                          // the pipeline's copy streams may still hold the slots
            FFCU_CHECK(cudaStreamSynchronize(c->s_in));
            FFCU_CHECK(cudaStreamSynchronize(c->s_out));
            c->lean_last = true;
        }
        FFCU_CHECK(cudaMemcpyAsync(c->in_slot[slot], host_in, (size_t)n * bytes_per_face, cudaMemcpyHostToDevice, c->stream));
        c->d_in = c->in_slot[slot]; c->d_out = c->out_slot[slot];
        c->in_u8 = u8;
        int rc = run_forward(c, n, slot);
        c->in_u8 = false;
        if (rc != 0) return rc;
        FFCU_CHECK(cudaMemcpyAsync(host_out, c->out_slot[slot], (size_t)n * 512 * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
        FFCU_CHECK(cudaMemcpyAsync(c->h_err, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
        c->err_copied = true;
        c->seq++;
        return 0;
    }
    if (c->lean_last) {                               // back to the pipeline: the compute stream owns the slots until it drains
        FFCU_CHECK(cudaStreamSynchronize(c->stream));
        c->lean_last = false;
    }
    // copy-in stream: the slot is free once the forward that last read it has finished
    if (reused) FFCU_CHECK(cudaStreamWaitEvent(c->s_in, c->ev_compute_done[slot], 0));
    FFCU_CHECK(cudaMemcpyAsync(c->in_slot[slot], host_in, (size_t)n * bytes_per_face, cudaMemcpyHostToDevice, c->s_in));
    FFCU_CHECK(cudaEventRecord(c->ev_in_ready[slot], c->s_in));
    // compute stream: needs the input, and the output slot drained by the copy-out of two steps ago
    FFCU_CHECK(cudaStreamWaitEvent(c->stream, c->ev_in_ready[slot], 0));
    if (reused) FFCU_CHECK(cudaStreamWaitEvent(c->stream, c->ev_out_copied[slot], 0));
    c->d_in = c->in_slot[slot]; c->d_out = c->out_slot[slot];
    c->in_u8 = u8;
    int rc = run_forward(c, n, slot);
    c->in_u8 = false;
    if (rc != 0) return rc;
    FFCU_CHECK(cudaEventRecord(c->ev_compute_done[slot], c->stream));
    // copy-out stream
    FFCU_CHECK(cudaStreamWaitEvent(c->s_out, c->ev_compute_done[slot], 0));
    FFCU_CHECK(cudaMemcpyAsync(host_out, c->out_slot[slot], (size_t)n * 512 * sizeof(float), cudaMemcpyDeviceToHost, c->s_out));
    FFCU_CHECK(cudaEventRecord(c->ev_out_copied[slot], c->s_out));
    c->seq++;
    return 0;
}

extern "C" int ffcu_submit(ffcu_ctx* c, const float* host_in, int n, float* host_out)
{
    return submit_impl(c, host_in, 37632 * sizeof(float), false, n, host_out);
}

extern "C" int ffcu_submit_u8(ffcu_ctx* c, const uint8_t* host_pixels, int n, float* host_out)
{
    return submit_impl(c, host_pixels, 37632, true, n, host_out);
}

extern "C" int ffcu_wait(ffcu_ctx* c)
{
    if (!c) return -1;
    FFCU_CHECK(cudaSetDevice(c->device));
    if (c->lean_last && c->err_copied) {
        FFCU_CHECK(cudaStreamSynchronize(c->stream));    // the error word's copy was queued behind the forward
    } else {
        FFCU_CHECK(cudaStreamSynchronize(c->s_in));
        FFCU_CHECK(cudaMemcpyAsync(c->h_err, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
        FFCU_CHECK(cudaStreamSynchronize(c->stream));
        FFCU_CHECK(cudaStreamSynchronize(c->s_out));
    }
    c->err_copied = false;
    if (*c->h_err != 0) {
        ffcu_set_error("device reported error word %d (a bounded wait inside a kernel ran out)", *c->h_err);
        int e = *c->h_err;
        cudaMemsetAsync(c->d_err, 0, sizeof(int), c->stream);
        // a launch that gave up may have left partial sums or tickets behind
        cudaMemsetAsync(c->d_fc_scratch, 0, (FFCU_FC_SMALL_TICKETS + FFCU_FC_SMALL_MAX_BATCH * 512) * sizeof(int), c->stream);
        cudaMemsetAsync(c->d_fc_tc_scratch, 0, ((size_t)FFCU_FC_TC_TICKETS + (size_t)c->fc_tc_rows * 512) * sizeof(int), c->stream);
        return 1000 + e;
    }
    return 0;
}

extern "C" int ffcu_trace(ffcu_ctx* c, const float* host_in, int n, float* host_out,
                          ffcu_trace_fn fn, void* user)
{
    if (!c || !c->finalized || !host_in || !host_out || n < 1 || n > c->max_batch) return -1;
    FFCU_CHECK(cudaSetDevice(c->device));
    size_t max_elems = (size_t)n * c->bytes_per_face;
    std::vector<uint8_t> host(max_elems * 4);
    int32_t* d_acc = nullptr;
    FFCU_CHECK(cudaMalloc(&d_acc, max_elems * sizeof(int32_t)));
    int rc = 0;
    {
        cudaError_t e = cudaMemcpyAsync(c->d_in, host_in, (size_t)n * 37632 * sizeof(float), cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) { ffcu_set_error("ffcu_trace: input copy failed: %s", cudaGetErrorString(e)); cudaFree(d_acc); return -100; }
    }
    for (size_t k = 0; k < c->layers.size() && rc == 0; k++) {
        const ffcu_layer& d = c->layers[k].d;
        rc = launch_layer(c, k, n, d.kind == FFCU_CONV ? d_acc : nullptr, true);
        if (rc != 0) break;
        rc = ffcu_wait(c);
        if (rc != 0 || !fn) continue;
        if (d.kind == FFCU_QUANT) {
            size_t npix = (size_t)n * d.H * d.W;
            cudaMemcpy(host.data(), c->bufs[d.dst_buf], npix * 4, cudaMemcpyDeviceToHost);
            std::vector<int8_t> q(npix * 3);     // dump in the reference's 3-channel layout
            for (size_t p = 0; p < npix; p++)
                for (int ch = 0; ch < 3; ch++) q[p * 3 + ch] = (int8_t)host[p * 4 + ch];
            fn(user, d.op_index, 'Q', q.data(), npix * 3);
        } else if (d.kind == FFCU_CONV) {
            size_t ne = (size_t)n * d.Ho * d.Wo * d.Cout;
            cudaMemcpy(host.data(), d_acc, ne * 4, cudaMemcpyDeviceToHost);
            fn(user, d.op_index, 'A', host.data(), ne);
            cudaMemcpy(host.data(), c->bufs[d.dst_buf], ne, cudaMemcpyDeviceToHost);
            fn(user, d.op_index, 'O', host.data(), ne);
            if (d.bn2_dst_buf >= 0) {       // BN fused as the conv's second output
                cudaMemcpy(host.data(), c->bufs[d.bn2_dst_buf], ne, cudaMemcpyDeviceToHost);
                fn(user, d.bn2_op_index, 'B', host.data(), ne);
            }
        } else if (d.kind == FFCU_BN) {
            size_t ne = (size_t)n * d.H * d.W * d.Cout;
            cudaMemcpy(host.data(), c->bufs[d.dst_buf], ne, cudaMemcpyDeviceToHost);
            fn(user, d.op_index, 'B', host.data(), ne);
        } else if (d.kind == FFCU_FC) {
            cudaMemcpy(host.data(), c->d_out, (size_t)n * 512 * 4, cudaMemcpyDeviceToHost);
            fn(user, d.op_index, 'F', host.data(), (size_t)n * 512);
        }
    }
    if (rc == 0) {
        cudaMemcpy(host_out, c->d_out, (size_t)n * 512 * sizeof(float), cudaMemcpyDeviceToHost);
        if (cudaGetLastError() != cudaSuccess) rc = -100;
    }
    cudaFree(d_acc);
    return rc;
}

extern "C" int ffcu_bench_resident(ffcu_ctx* c, const float* host_in, int n, int iters, float* ms)
{
    if (!c || !c->finalized || !host_in || !ms || n < 1 || n > c->max_batch || iters < 1) return -1;
    FFCU_CHECK(cudaSetDevice(c->device));
    c->d_in = c->in_slot[0]; c->d_out = c->out_slot[0];
    FFCU_CHECK(cudaMemcpyAsync(c->d_in, host_in, (size_t)n * 37632 * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    cudaEvent_t e0, e1;
    FFCU_CHECK(cudaEventCreate(&e0));
    FFCU_CHECK(cudaEventCreate(&e1));
    FFCU_CHECK(cudaStreamSynchronize(c->stream));
    FFCU_CHECK(cudaEventRecord(e0, c->stream));
    int rc = 0;
    for (int it = 0; it < iters && rc == 0; it++) rc = run_forward(c, n, 0);
    FFCU_CHECK(cudaEventRecord(e1, c->stream));
    int wrc = ffcu_wait(c);
    if (rc == 0) rc = wrc;
    if (rc == 0) FFCU_CHECK(cudaEventElapsedTime(ms, e0, e1));
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return rc;
}

extern "C" int ffcu_layer_count(const ffcu_ctx* c) { return c ? (int)c->layers.size() : 0; }

extern "C" int ffcu_layer_info(const ffcu_ctx* c, int k, ffcu_layer* out, int* uses_tc)
{
    if (!c || !out || k < 0 || k >= (int)c->layers.size()) return -1;
    *out = c->layers[k].d;
    if (uses_tc) *uses_tc = (c->layers[k].tc || c->layers[k].stem_tc) ? 1 : 0;
    return 0;
}

extern "C" int ffcu_bench_layers(ffcu_ctx* c, const float* host_in, int n, int iters, float* ms, int cap)
{
    if (!c || !c->finalized || !host_in || !ms || n < 1 || n > c->max_batch || iters < 1) return -1;
    const int nl = (int)c->layers.size();
    if (cap < nl) { ffcu_set_error("ffcu_bench_layers: ms[] too small"); return -1; }
    FFCU_CHECK(cudaSetDevice(c->device));
    FFCU_CHECK(cudaMemcpyAsync(c->d_in, host_in, (size_t)n * 37632 * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    int rc = launch_forward(c, n);
    if (rc != 0) return rc;
    std::vector<cudaEvent_t> ev(2 * nl);
    for (auto& e : ev) FFCU_CHECK(cudaEventCreate(&e));
    for (int k = 0; k < nl && rc == 0; k++) {
        DevLayer& M = c->layers[k];
        // a stride-2 conv that shares its launch with the block's shortcut at this batch is timed as the forward runs
        // it: the pair's one launch under the conv, nothing under the shortcut
        const bool pair = M.sc && k + 1 < nl && ffcu_tc_pick_bn(M.d, n, c->device, 1) == 64;
        FFCU_CHECK(cudaEventRecord(ev[2 * k], c->stream));
        for (int it = 0; it < iters && rc == 0; it++) {
            if (pair) {
                DevLayer& S = c->layers[k + 1];
                rc = ffcu_sc_launch(M.sc, n, c->mode, M.epi, S.epi, c->bufs[M.d.dst_buf], M.sc_write_main, c->bufs[S.d.dst_buf],
                                    S.d.bn2_dst_buf >= 0 ? c->bufs[S.d.bn2_dst_buf] : nullptr, c->d_err, c->stream);
            } else rc = launch_layer(c, k, n, nullptr);
        }
        FFCU_CHECK(cudaEventRecord(ev[2 * k + 1], c->stream));
        if (pair) {
            k++;
            FFCU_CHECK(cudaEventRecord(ev[2 * k], c->stream));
            FFCU_CHECK(cudaEventRecord(ev[2 * k + 1], c->stream));
        }
    }
    int wrc = ffcu_wait(c);
    if (rc == 0) rc = wrc;
    for (int k = 0; k < nl && rc == 0; k++) FFCU_CHECK(cudaEventElapsedTime(&ms[k], ev[2 * k], ev[2 * k + 1]));
    for (auto& e : ev) cudaEventDestroy(e);
    return rc == 0 ? nl : rc;
}

// ---------------------------------------------------------------------------
// one conv layer on caller-supplied host tensors (single-layer parity tests)
// ---------------------------------------------------------------------------
static int conv_once_impl(int device, const ffcu_layer* l, int batch, int mode, int impl,
                          const int8_t* in, const int8_t* res, int32_t* acc_out, int8_t* out, int8_t* out_bn2,
                          int iters, float* ms)
{
    if (!l || !in || batch < 1 || l->kind != FFCU_CONV) { ffcu_set_error("ffcu_conv_once: bad arguments"); return -1; }
    FFCU_CHECK(cudaSetDevice(device));
    const size_t in_bytes = (size_t)batch * l->H * l->W * l->Cin_pad;
    const size_t out_elems = (size_t)batch * l->Ho * l->Wo * l->Cout;
    int8_t *d_in = nullptr, *d_res = nullptr, *d_out = nullptr, *d_w = nullptr, *d_out2 = nullptr, *d_lut = nullptr;
    int32_t* d_acc = nullptr; int* d_err = nullptr;
    float* tab[9] = {};
    cudaStream_t s = nullptr;
    TcPlan* plan = nullptr;
    const bool bn2 = out_bn2 && l->bn2_in_scale && l->bn2_scale && l->bn2_offset && l->bn2_inv_out;
    int rc = 0;
    // one exit: everything allocated so far is released whatever step failed
#define ONCE_TRY(expr)                                                                           \
    do {                                                                                         \
        cudaError_t _e = (expr);                                                                 \
        if (_e != cudaSuccess && rc == 0) {                                                      \
            ffcu_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            rc = -100;                                                                           \
        }                                                                                        \
    } while (0)
    if (bn2) ONCE_TRY(cudaMalloc(&d_out2, out_elems + 1024));
    ONCE_TRY(cudaMalloc(&d_in, in_bytes + 1024));
    ONCE_TRY(cudaMalloc(&d_out, out_elems + 1024));
    ONCE_TRY(cudaMalloc(&d_w, l->w_bytes + 1024));
    ONCE_TRY(cudaMalloc(&d_err, sizeof(int)));
    if (acc_out) ONCE_TRY(cudaMalloc(&d_acc, out_elems * 4));
    if (res) ONCE_TRY(cudaMalloc(&d_res, out_elems));
    if (rc == 0) {
        ONCE_TRY(cudaMemset(d_err, 0, sizeof(int)));
        ONCE_TRY(cudaMemset(d_w, 0, l->w_bytes + 1024));
        ONCE_TRY(cudaMemset(d_out, 0x55, out_elems + 1024));
        if (res) ONCE_TRY(cudaMemcpy(d_res, res, out_elems, cudaMemcpyHostToDevice));
        ONCE_TRY(cudaMemcpy(d_in, in, in_bytes, cudaMemcpyHostToDevice));
        ONCE_TRY(cudaMemcpy(d_w, l->w, l->w_bytes, cudaMemcpyHostToDevice));
    }
    const float* src[9] = {l->w_scale, l->bias, l->slope, l->res_scale, l->inv_out,
                           bn2 ? l->bn2_in_scale : nullptr, bn2 ? l->bn2_scale : nullptr,
                           bn2 ? l->bn2_offset : nullptr, bn2 ? l->bn2_inv_out : nullptr};
    for (int k = 0; k < 9 && rc == 0; k++)
        if (src[k]) {
            tab[k] = upload_f32(src[k], l->Cout);
            if (!tab[k]) { ffcu_set_error("ffcu_conv_once: table allocation or upload failed"); rc = -100; }
        }
    if (bn2 && rc == 0) {
        std::vector<int8_t> lut((size_t)l->Cout * 256);
        ff_bn_lut_build(l->bn2_in_scale, l->bn2_scale, l->bn2_offset, l->bn2_inv_out, l->Cout, lut.data());
        ONCE_TRY(cudaMalloc(&d_lut, lut.size()));
        if (rc == 0) ONCE_TRY(cudaMemcpy(d_lut, lut.data(), lut.size(), cudaMemcpyHostToDevice));
    }
    if (rc == 0) ONCE_TRY(cudaStreamCreate(&s));
    if (rc == 0) {
        EpiTables t{tab[0], tab[1], tab[2], tab[3], tab[4], tab[5], tab[6], tab[7], tab[8], d_lut};
        t.no_overflow = epilogue_cannot_overflow(l) ? 1 : 0;
        t.acc22 = accumulator_fits_22_bits(l) ? 1 : 0;
        if (impl == 0) {
            plan = ffcu_tc_plan(*l, batch, d_in, d_w, device, ffcu_tc_pick_bn(*l, batch, device));
            if (!plan) { ffcu_set_error("layer shape is not covered by the tensor-core kernel"); rc = -2; }
            else rc = ffcu_tc_launch(plan, batch, mode, t, d_res, d_acc, d_out, d_out2, d_err, s);
        } else {
            rc = ffcu_launch_conv_simt(*l, batch, mode, d_in, d_w, t, d_res, d_acc, d_out, d_out2, s);
        }
    }
    if (rc == 0) {
        cudaError_t e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) { ffcu_set_error("kernel failed: %s", cudaGetErrorString(e)); rc = -100; }
    }
    if (rc == 0 && iters > 0 && ms) {
        // timing: `iters` more launches of the same layer between two events on its stream
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        ONCE_TRY(cudaEventCreate(&e0));
        ONCE_TRY(cudaEventCreate(&e1));
        EpiTables t{tab[0], tab[1], tab[2], tab[3], tab[4], tab[5], tab[6], tab[7], tab[8], d_lut};
        t.no_overflow = epilogue_cannot_overflow(l) ? 1 : 0;
        t.acc22 = accumulator_fits_22_bits(l) ? 1 : 0;
        if (rc == 0) ONCE_TRY(cudaEventRecord(e0, s));
        for (int it = 0; it < iters && rc == 0; it++)
            rc = impl == 0 ? ffcu_tc_launch(plan, batch, mode, t, d_res, d_acc, d_out, d_out2, d_err, s)
                           : ffcu_launch_conv_simt(*l, batch, mode, d_in, d_w, t, d_res, d_acc, d_out, d_out2, s);
        if (rc == 0) ONCE_TRY(cudaEventRecord(e1, s));
        if (rc == 0) ONCE_TRY(cudaEventSynchronize(e1));
        float total = 0;
        if (rc == 0) ONCE_TRY(cudaEventElapsedTime(&total, e0, e1));
        if (rc == 0) *ms = total / iters;
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
    }
    if (rc == 0) {
        int herr = 0;
        ONCE_TRY(cudaMemcpy(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost));
        if (rc == 0 && herr) { ffcu_set_error("device reported error word %d (a bounded wait inside a kernel ran out)", herr); rc = 1000 + herr; }
    }
    if (rc == 0 && acc_out) ONCE_TRY(cudaMemcpy(acc_out, d_acc, out_elems * 4, cudaMemcpyDeviceToHost));
    if (rc == 0 && out) ONCE_TRY(cudaMemcpy(out, d_out, out_elems, cudaMemcpyDeviceToHost));
    if (rc == 0 && bn2) ONCE_TRY(cudaMemcpy(out_bn2, d_out2, out_elems, cudaMemcpyDeviceToHost));
#undef ONCE_TRY
    if (plan) ffcu_tc_free(plan);
    if (s) cudaStreamDestroy(s);
    cudaFree(d_lut); cudaFree(d_in); cudaFree(d_res); cudaFree(d_out); cudaFree(d_out2); cudaFree(d_w); cudaFree(d_acc); cudaFree(d_err);
    for (float* q : tab) cudaFree(q);
    return rc;
}

extern "C" int ffcu_conv_once(int device, const ffcu_layer* l, int batch, int mode, int impl,
                              const int8_t* in, const int8_t* res, int32_t* acc_out, int8_t* out, int8_t* out_bn2)
{
    return conv_once_impl(device, l, batch, mode, impl, in, res, acc_out, out, out_bn2, 0, nullptr);
}

extern "C" int ffcu_conv_bench(int device, const ffcu_layer* l, int batch, int mode, int impl,
                               const int8_t* in, const int8_t* res, int8_t* out, int8_t* out_bn2, int iters, float* ms)
{
    if (iters < 1 || !ms) { ffcu_set_error("ffcu_conv_bench: bad arguments"); return -1; }
    return conv_once_impl(device, l, batch, mode, impl, in, res, nullptr, out, out_bn2, iters, ms);
}
