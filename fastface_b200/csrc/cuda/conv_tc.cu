// conv_tc.cu -- host side of the tensor-core convolution: per-layer kernel choice, tile
// geometry, TMA descriptors, launch.  The kernels live in conv_tc_{generic,ws,pair,k32}.cu.
#include "conv_tc_common.cuh"
#include <vector>

// ---------------------------------------------------------------------------
// host side: tile geometry, tensor maps, launch
// ---------------------------------------------------------------------------
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode()
{
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)p;
    }
    return fn;
}

struct TcGeom { int TW, TH, TB; CUtensorMap mapA; bool valid; };

struct TcPlan {
    ffcu_layer d;
    int max_batch;
    int BN, KC, stages, smem_bytes;
    bool out_f32;
    const int8_t* d_in;
    CUtensorMap mapB;
    int n_sm;
    int group, pair_group;   // K blocks per pipeline stage
    int lut_bytes;           // shared memory for the fused BN's byte table
    int ntab;                // per-channel tables in shared memory (5, or 9 with an arithmetic fused BN)
    TcGeom geoms[8];
    int n_geoms;
    bool pair;               // CTA-pair kernel (cta_group::2) for >= 128 input channels
    CUtensorMap mapB_half;   // box {128, BN/2}
    int pair_stages, pair_smem_bytes;
    bool wsp;                // flat-pitch weight-stationary pair kernel (128 -> 128 3x3 stride-1 layers, 28x28 maps)
    CUtensorMap mapA_wsp;    // box {128, W + 2, 8, 1}
    int wsp_P, wsp_tiles_per_image, wsp_stages, wsp_smem_bytes;
    bool ws;                 // weight-stationary kernel (64-channel 3x3 stride-1 layers)
    CUtensorMap mapA_ws;     // box {64, 8, 18, 1}
    int ws_stages, ws_smem_bytes;
};

// Output-tile shape {TW, TH, TB} with TW*TH*TB = 128 that wastes the fewest rows for this
// feature-map size and batch; ties go to the widest tile.
static void pick_geometry(int Wo, int Ho, int batch, int* TW, int* TH, int* TB)
{
    double best = 1e300; int bw = 1, bh = 1, bb = 128;
    for (int tw = 128; tw >= 1; tw >>= 1)
        for (int th = 128 / tw; th >= 1; th >>= 1) {
            int tb = 128 / (tw * th);
            double padded = (double)((Wo + tw - 1) / tw * tw) * ((Ho + th - 1) / th * th) * ((batch + tb - 1) / tb * tb);
            if (padded < best) { best = padded; bw = tw; bh = th; bb = tb; }
        }
    *TW = bw; *TH = bh; *TB = bb;
}

static bool encode_A(const TcPlan* p, TcGeom* g)
{
    encode_tiled_fn enc = get_encode();
    if (!enc) { ffcu_set_error("cuTensorMapEncodeTiled is not available"); return false; }
    const ffcu_layer& d = p->d;
    const cuuint64_t Cp = (cuuint64_t)d.Cin_pad;
    cuuint64_t dims[4] = {Cp, (cuuint64_t)d.W, (cuuint64_t)d.H, (cuuint64_t)p->max_batch};
    cuuint64_t strides[3] = {Cp, Cp * d.W, Cp * d.W * d.H};
    cuuint32_t box[4] = {(cuuint32_t)p->KC, (cuuint32_t)(g->TW * d.stride), (cuuint32_t)(g->TH * d.stride), (cuuint32_t)g->TB};
    cuuint32_t estr[4] = {1, (cuuint32_t)d.stride, (cuuint32_t)d.stride, 1};
    if (d.stride > 1) {      // a unit-extent dimension needs no traversal stride
        if (g->TW == 1) { box[1] = 1; estr[1] = 1; }
        if (g->TH == 1) { box[2] = 1; estr[2] = 1; }
    }
    CUresult r = enc(&g->mapA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)p->d_in, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     p->KC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(A) failed: %d", (int)r); return false; }
    return true;
}

// Column-tile width for a call of `batch` faces.  BN = min(256, Cout) when the batch fills the
// machine.  A batch that yields fewer tiles than SMs (latency use: one face is 2 row tiles on the
// 14x14 maps) takes narrower column tiles, so that Cout / BN times as many SMs share the layer's
// weight stream instead of one SM reading all of it.  $FF_TC_BN: 64 / 128 / 256 pins the tile
// where it divides Cout; "wide" keeps the widest tile at any batch.  The tile is halved while the launch would
// fill less than 1 / fill_div of the SMs: half (the default, $FF_TC_BN_FILL) measured best at batch 16-128, where
// a wider tile on half the SMs beats twice the CTAs each streaming the same activations again; the fused
// stride-2 + shortcut launch (64 columns only) asks with fill_div = 1, the rule it was measured with.
int ffcu_tc_pick_bn(const ffcu_layer& L, int batch, int device, int fill_div)
{
    int bn = L.Cout >= 256 ? 256 : L.Cout;
    const char* bn_env = getenv("FF_TC_BN");
    if (bn_env) {
        int v = atoi(bn_env);
        if ((v == 64 || v == 128 || v == 256) && L.Cout % v == 0) bn = v;
        return bn;
    }
    static int n_sm_dev[64] = {};
    int& n_sm = n_sm_dev[device & 63];
    if (!n_sm && cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) n_sm = 148;
    static int fill_env = -1;
    if (fill_env < 0) { const char* e = getenv("FF_TC_BN_FILL"); fill_env = (e && atoi(e) >= 1 && atoi(e) <= 4) ? atoi(e) : 2; }
    if (fill_div < 1) fill_div = fill_env;
    const long long rows = (L.kind == FFCU_FC) ? (long long)batch : (long long)batch * L.Ho * L.Wo;
    const long long m_tiles = (rows + TC_TILE_M - 1) / TC_TILE_M;
    while (bn > 64 && L.Cout % (bn / 2) == 0 && m_tiles * (L.Cout / bn) * fill_div < n_sm) bn /= 2;
    return bn;
}

// One-shot fault injection for the timeout-path test (ffcu_test_arm_timeout): consumed by the
// next launch of the one-CTA per-tap kernel.
static int g_test_drop_stage = -1;
static long long g_test_full_wait = 0;

extern "C" void ffcu_test_arm_timeout(int drop_stage, long long full_wait_cycles)
{
    g_test_drop_stage = drop_stage;
    g_test_full_wait = full_wait_cycles;
}

TcPlan* ffcu_tc_plan(const ffcu_layer& L, int max_batch, const int8_t* d_in, const int8_t* d_w, int device, int bn)
{
    if (L.kind != FFCU_CONV && L.kind != FFCU_FC) return nullptr;
    const int Cp = L.Cin_pad;
    if (Cp % 64 != 0 || L.Cout % 64 != 0 || L.Cout > TC_MAX_COUT) return nullptr;
    if (L.stride < 1 || L.stride > 2 || L.Kh * L.Kw > 9) return nullptr;
    if (L.stride == 2 && getenv("FF_TC_STRIDE2") && atoi(getenv("FF_TC_STRIDE2")) == 0) return nullptr;
    if ((bn != 64 && bn != 128 && bn != 256) || L.Cout % bn != 0) return nullptr;
    encode_tiled_fn enc = get_encode();
    if (!enc) return nullptr;
    TcPlan* p = new TcPlan();
    p->d = L; p->max_batch = max_batch; p->d_in = d_in; p->n_geoms = 0;
    p->out_f32 = (L.kind == FFCU_FC);
    p->KC = (Cp % 128 == 0) ? 128 : 64;
    p->BN = bn;
    // fused BN: a byte table in shared memory for tiles up to $FF_TC_BNLUT_MAX channels wide, arithmetic beyond
    // (default: the table everywhere; measured 2 - 3 % faster per step than arithmetic for the wide tiles although
    // it costs those a pipeline stage)
    const char* lm = getenv("FF_TC_BNLUT_MAX");
    const int lut_max = lm ? atoi(lm) : 256;
    const int lut_bytes = (L.kind == FFCU_CONV && L.bn2_dst_buf >= 0 && p->BN <= lut_max) ? p->BN * 256 : 0;
    const int ntab = (L.kind == FFCU_CONV && L.bn2_dst_buf >= 0 && !lut_bytes) ? 9 : 5;
    p->ntab = ntab;
    const int fixed = ntab * TC_MAX_COUT * 4 + (int)sizeof(TcShared) + 1024 + lut_bytes;
    p->lut_bytes = lut_bytes;
    const int kblocks = L.Kh * L.Kw * (Cp / p->KC);
    const char* genv = getenv("FF_TC_GROUP");
    const int gmax = genv ? atoi(genv) : 8;
    // K blocks per stage.  One barrier hand-shake costs the single-thread producer / issuer
    // loops about 500 cycles whatever it moves, so a stage should hold >= ~768 cycles of MMA work
    // (one block = 128 x BN x KC MACs at 8192 MACs/cycle); the group must divide the K loop and
    // leave at least two stages.
    const int blk_cycles = 2 * p->BN * p->KC / 128;
    const int g_target = (768 + blk_cycles - 1) / blk_cycles;
    auto pick_group = [&](int sub_bytes, int* stages_out) {
        int best_g = 1;
        for (int g = 2; g <= gmax && g <= 8; g++) {
            if (kblocks % g) continue;
            if ((232448 - fixed) / (g * sub_bytes) < 2) break;
            best_g = g;
            if (g >= g_target) break;
        }
        int st = (232448 - fixed) / (best_g * sub_bytes);
        if (st > TC_MAX_STAGES) st = TC_MAX_STAGES;
        *stages_out = st;
        return best_g;
    };
    const int sub_bytes = (TC_TILE_M + p->BN) * p->KC;
    int stages = 0;
    p->group = pick_group(sub_bytes, &stages);
    if (stages < 2) { delete p; return nullptr; }
    p->stages = stages;
    p->smem_bytes = stages * p->group * sub_bytes + fixed;
    cudaDeviceGetAttribute(&p->n_sm, cudaDevAttrMultiProcessorCount, device);
    // weights: [Cout][taps*Cp] K-major
    cuuint64_t Ktot = (cuuint64_t)L.Kh * L.Kw * Cp;
    // 4-D like the activation map so one cp.async.bulk.tensor.4d instruction serves both operands
    cuuint64_t dims[4] = {Ktot, (cuuint64_t)L.Cout, 1, 1};
    cuuint64_t strides[3] = {Ktot, Ktot * L.Cout, Ktot * L.Cout};
    cuuint32_t box[4] = {(cuuint32_t)p->KC, (cuuint32_t)p->BN, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&p->mapB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_w, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     p->KC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(B) failed: %d", (int)r); delete p; return nullptr; }
    // CTA-pair variant
    p->pair = false;
    const char* pair_env = getenv("FF_TC_PAIR");
    if (p->KC == 128 && (p->BN == 128 || p->BN == 256) && !(pair_env && pair_env[0] == '0')) {
        cuuint32_t hbox[4] = {128, (cuuint32_t)(p->BN / 2), 1, 1};
        r = enc(&p->mapB_half, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_w, dims, strides, hbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS) {
            const int sb = (TC_TILE_M + p->BN / 2) * 128;
            int st = 0;
            p->pair_group = pick_group(sb, &st);
            if (st == 2 && p->pair_group > 1 && lut_bytes && !genv) {
                // the fused BN's byte table has taken the third stage: four (or more) stages of one K block keep more
                // bytes in flight than two of several (measured on the 14x14 / 7x7 residual + BN layers: -1.6 % / -3 %)
                int st1 = (232448 - fixed) / sb;
                if (st1 > TC_MAX_STAGES) st1 = TC_MAX_STAGES;
                if (st1 >= 4) { p->pair_group = 1; st = st1; }
            }
            if (st >= 2) { p->pair = true; p->pair_stages = st; p->pair_smem_bytes = st * p->pair_group * sb + fixed; }
        }
    }
    // flat-pitch weight-stationary pair variant: all nine taps of a 128 -> 128 layer resident, one box per tile
    p->wsp = false;
    const char* wsp_env = getenv("FF_TC_WSP");
    if (p->pair && L.kind == FFCU_CONV && Cp == 128 && L.Cout == 128 && p->BN == 128 && L.Kh == 3 && L.Kw == 3 &&
        L.stride == 1 && L.pad == 1 && !(wsp_env && wsp_env[0] == '0')) {
        const int P = L.W + 2;
        const int rows_needed = (TC_TILE_M - 1 + P - 1) / P + 1 + 2;       // rows a tile's lines span, plus one above and below
        if (rows_needed <= WSP_BOX_ROWS && P <= 256) {
            cuuint64_t adims[4] = {128, (cuuint64_t)L.W, (cuuint64_t)L.H, (cuuint64_t)max_batch};
            cuuint64_t astr[3] = {128, (cuuint64_t)128 * L.W, (cuuint64_t)128 * L.W * L.H};
            cuuint32_t abox[4] = {128, (cuuint32_t)P, WSP_BOX_ROWS, 1};
            cuuint32_t aes[4] = {1, 1, 1, 1};
            r = enc(&p->mapA_wsp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_in, adims, astr, abox, aes,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r == CUDA_SUCCESS) {
                const int a_stride = (WSP_GUARD_BYTES + P * WSP_BOX_ROWS * 128 + 1023) & ~1023;
                const int wbytes = 9 * (p->BN / 2) * 128;
                int st = (232448 - wbytes - fixed) / a_stride;
                if (st > 4) st = 4;
                // Two issuer warps take alternate tiles and find their ring slot from the tile's index: with an
                // odd ring a warp's "this slot's data has landed" test would look at a slot the OTHER warp's
                // previous tile may still be waiting on, and a parity test cannot tell "one fill behind" from
                // "this fill done".  An even ring keeps every slot a warp tests behind one of its own tiles.
                st &= ~1;
                if (st >= 2) {
                    p->wsp = true; p->wsp_P = P; p->wsp_tiles_per_image = (L.H * P + TC_TILE_M - 1) / TC_TILE_M;
                    p->wsp_stages = st; p->wsp_smem_bytes = wbytes + st * a_stride + fixed;
                }
            }
        }
    }
    // weight-stationary variant
    p->ws = false;
    const char* ws_env = getenv("FF_TC_WS");
    if (L.kind == FFCU_CONV && Cp == 64 && L.Kh == 3 && L.Kw == 3 && L.stride == 1 && L.pad == 1 &&
        (L.Cout == 64 || L.Cout == 128) && p->BN == L.Cout && L.W % WS_TW == 0 && L.H >= WS_TH &&
        !(ws_env && ws_env[0] == '0')) {
        cuuint64_t adims[4] = {64, (cuuint64_t)L.W, (cuuint64_t)L.H, (cuuint64_t)max_batch};
        cuuint64_t astr[3] = {64, (cuuint64_t)64 * L.W, (cuuint64_t)64 * L.W * L.H};
        cuuint32_t abox[4] = {64, WS_PITCH, WS_TH + 2, 1};
        cuuint32_t aes[4] = {1, 1, 1, 1};
        r = enc(&p->mapA_ws, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_in, adims, astr, abox, aes,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS) {
            const int wbytes = 9 * p->BN * 64;
            int st = (232448 - wbytes - fixed) / WS_A_BYTES;
            if (st > TC_MAX_STAGES) st = TC_MAX_STAGES;
            st &= ~1;                                     // two issuer warps on alternate tiles: the ring must be even (see above)
            if (st >= 2) { p->ws = true; p->ws_stages = st; p->ws_smem_bytes = wbytes + st * WS_A_BYTES + fixed; }
        }
    }
    return p;
}

void ffcu_tc_free(TcPlan* p) { delete p; }

// Epilogue warps per set for a launch whose CTAs each see about tiles_per_cta tiles of bn columns.
// Narrow tiles at large batch: four (per-tile bookkeeping spread over twice the elements); otherwise
// eight (half the tile latency).  $FF_TC_WPS64 / $FF_TC_WPS128 = 4 or 8 override.
static int tc_epi_wps(int bn, int tiles_per_cta)
{
    static int w64 = -1, w128 = -1;
    if (w64 < 0) { const char* e = getenv("FF_TC_WPS64"); w64 = (e && (atoi(e) == 4 || atoi(e) == 8)) ? atoi(e) : 0; }
    if (w128 < 0) { const char* e = getenv("FF_TC_WPS128"); w128 = (e && (atoi(e) == 4 || atoi(e) == 8)) ? atoi(e) : 0; }
    if (bn == 64) return w64 ? w64 : (tiles_per_cta >= 8 ? 4 : 8);
    if (bn == 128) return w128 ? w128 : 8;
    return 8;
}

static int g_test_fc_drop_step = -1;
static long long g_test_fc_wait = 0;

extern "C" void ffcu_test_arm_fc_timeout(int drop_step, long long wait_cycles)
{
    g_test_fc_drop_step = drop_step;
    g_test_fc_wait = wait_cycles;
}

// The FC as a split-K GEMM (conv_tc_fc.cu): `scratch` = tiles' tickets (FFCU_FC_TC_TICKETS ints) followed by
// [rows][N] int32 sums, all zero between calls.  Returns 1 when this plan / batch does not take that kernel
// (the caller then launches the one-CTA-per-tile form), 0 on success, < 0 on error.
int ffcu_fc_tc_launch(const TcPlan* cp, int batch, int mode, const EpiTables& t, float* out, int* scratch, int scratch_rows,
                      int* d_err, cudaStream_t s)
{
    TcPlan* p = const_cast<TcPlan*>(cp);
    static int on = -1;
    if (on < 0) { const char* e = getenv("FF_FC_SPLITK"); on = (e && e[0] == '0') ? 0 : 1; }
    if (!on || !scratch || !p->out_f32 || p->BN != 64 || p->KC != 128 || p->pair || p->ws || p->wsp) return 1;
    const ffcu_layer& d = p->d;
    const int kblocks = d.Cin_pad / 128;
    const int tiles_n = d.Cout / 64, tiles_m = (batch + TC_TILE_M - 1) / TC_TILE_M;
    if (batch < 1 || batch > p->max_batch || d.Cin_pad % 128 != 0 || tiles_m * TC_TILE_M > scratch_rows ||
        tiles_m * tiles_n > FFCU_FC_TC_TICKETS) return 1;
    // K ranges: the most that divide the K loop, leave two K blocks per CTA and keep the grid within the SMs
    int splits = 1;
    for (int sp = 2; sp <= kblocks / 2; sp++)
        if (kblocks % sp == 0 && tiles_n * tiles_m * sp <= p->n_sm) splits = sp;
    { const char* e = getenv("FF_FC_SPLITS"); const int v = e ? atoi(e) : 0; if (v >= 1 && v <= kblocks / 2 && kblocks % v == 0) splits = v; }
    const int bps = kblocks / splits;
    if (d.Wo != 1 || d.Ho != 1 || d.W != 1 || d.H != 1) return 1;
    const int TW = 1, TH = 1, TB = TC_TILE_M;              // a row tile = 128 consecutive faces
    TcGeom* g = nullptr;
    for (int i = 0; i < p->n_geoms; i++)
        if (p->geoms[i].TW == TW && p->geoms[i].TH == TH && p->geoms[i].TB == TB) g = &p->geoms[i];
    if (!g) {
        if (p->n_geoms == 8) p->n_geoms = 0;
        g = &p->geoms[p->n_geoms];
        g->TW = TW; g->TH = TH; g->TB = TB;
        if (!encode_A(p, g)) return -1;
        p->n_geoms++;
    }
    FcTcParams prm = {};
    prm.w_scale = t.w_scale; prm.bias = t.bias; prm.out = out;
    prm.tickets = scratch; prm.sums = scratch + FFCU_FC_TC_TICKETS; prm.err = d_err;
    prm.batch = batch; prm.N = d.Cout;
    prm.tiles_n = tiles_n; prm.tiles_m = tiles_m; prm.splits = splits; prm.blocks_per_split = bps;
    prm.group = (bps % 2 == 0) ? 2 : 1;
    const int sub = (TC_TILE_M + 64) * 128;
    int st = (232448 - (int)sizeof(TcShared) - 2048) / (prm.group * sub);
    if (st > TC_MAX_STAGES) st = TC_MAX_STAGES;
    if (st > bps / prm.group) st = bps / prm.group;
    if (st < 1) return 1;
    prm.stages = st;
    prm.drop_step = -1; prm.wait_cycles = TC_WAIT_CYCLES;
    if (g_test_fc_drop_step >= 0) {                          // armed for this one launch by the timeout test
        prm.drop_step = g_test_fc_drop_step;
        if (g_test_fc_wait > 0) prm.wait_cycles = g_test_fc_wait;
        g_test_fc_drop_step = -1; g_test_fc_wait = 0;
    }
    const int smem = st * prm.group * sub + (int)sizeof(TcShared) + 2048;
    return tc_launch_fc(mode, tiles_n * tiles_m * splits, smem, s, g->mapA, p->mapB, prm);
}

int ffcu_tc_launch(const TcPlan* cp, int batch, int mode, const EpiTables& t, const int8_t* res,
                   int32_t* acc_out, void* out, int8_t* out_bn2, int* d_err, cudaStream_t s)
{
    TcPlan* p = const_cast<TcPlan*>(cp);
    if (batch < 1 || batch > p->max_batch) { ffcu_set_error("tc launch: batch out of range"); return -1; }
    const ffcu_layer& d = p->d;
#ifdef FF_TC_TIMING
    static int dbg = -1;
    if (dbg < 0) { const char* e = getenv("FF_TC_DBG"); dbg = e ? atoi(e) : 0; }
#endif
    const bool has_res = res && t.res_scale, has_slope = t.slope != nullptr, has_bn2 = out_bn2 && t.bn_in;
    int epi = EPI_RUNTIME;
    if (p->out_f32 || (!has_res && !has_slope && !has_bn2)) epi = EPI_PLAIN;
    else if (has_slope && !has_res && !has_bn2) epi = EPI_SLOPE;
    else if (has_res && has_bn2 && !has_slope) epi = EPI_RES_BN;
    else if (has_res && !has_bn2 && !has_slope) epi = EPI_RES;
    // the specialised variants carry no accumulator dump, no out-of-range conversion check and no
    // arithmetic fused BN: a launch that needs one of those takes the general variant
    if (!p->out_f32 && (acc_out || !t.no_overflow || (has_bn2 && !p->lut_bytes))) epi = EPI_RUNTIME;
    // the specialised variants of the 64-input-channel kernels convert the accumulator without the conversion
    // unit, which is exact below 2^22: a layer without that bound takes the general variant too
    if (!p->out_f32 && p->KC == 64 && !t.acc22) epi = EPI_RUNTIME;
    if (p->ws) {
        TcParams prm = {};
        prm.t = t; prm.res = res; prm.acc_out = acc_out; prm.out = out; prm.err = d_err;
        prm.out2 = (out_bn2 && t.bn_in) ? out_bn2 : nullptr;
        prm.batch = batch; prm.Ho = d.Ho; prm.Wo = d.Wo; prm.Cout = d.Cout;
        prm.taps = 9; prm.Kw = 3; prm.Cp = 64; prm.cin_blocks = 1; prm.stride = 1; prm.pad = 1;
        prm.TW = WS_TW; prm.TH = WS_TH; prm.TB = 1;
        prm.tiles_w = d.Wo / WS_TW; prm.tiles_h = (d.Ho + WS_TH - 1) / WS_TH; prm.tiles_b = batch; prm.tiles_n = 1;
        prm.total_tiles = prm.tiles_w * prm.tiles_h * batch;
        prm.stages = p->ws_stages; prm.group = 1; prm.lut_bytes = p->lut_bytes; prm.ntab = p->ntab;
        prm.full_wait = TC_WAIT_CYCLES; prm.drop_stage = -1;
#ifdef FF_TC_TIMING
        prm.dbg = dbg;
#endif
        int grid = prm.total_tiles < p->n_sm ? prm.total_tiles : p->n_sm;
        prm.epi_wps = tc_epi_wps(p->BN, prm.total_tiles / grid);
        return tc_launch_ws(p->BN, mode, epi, grid, p->ws_smem_bytes, s, p->mapA_ws, p->mapB, prm);
    }
    if (p->wsp) {
        TcParams prm = {};
        prm.t = t; prm.res = res; prm.acc_out = acc_out; prm.out = out; prm.err = d_err;
        prm.out2 = (out_bn2 && t.bn_in) ? out_bn2 : nullptr;
        prm.batch = batch; prm.Ho = d.Ho; prm.Wo = d.Wo; prm.Cout = d.Cout;
        prm.taps = 9; prm.Kw = 3; prm.Cp = 128; prm.cin_blocks = 1; prm.stride = 1; prm.pad = 1;
        prm.TW = TC_TILE_M; prm.TH = 1; prm.TB = 1;        // not used for the mapping: flat_P is set
        prm.flat_P = p->wsp_P;
        const int images = (batch + 1) & ~1;               // a pair takes one tile of two consecutive images
        prm.tiles_w = images; prm.tiles_h = p->wsp_tiles_per_image; prm.tiles_b = 1; prm.tiles_n = 1;
        prm.total_tiles = (images / 2) * p->wsp_tiles_per_image;
        prm.stages = p->wsp_stages; prm.group = 1; prm.lut_bytes = p->lut_bytes; prm.ntab = p->ntab;
        prm.full_wait = TC_WAIT_CYCLES; prm.drop_stage = -1;
#ifdef FF_TC_TIMING
        prm.dbg = dbg;
#endif
        const int max_pairs = p->n_sm / 2;
        const int npairs = prm.total_tiles < max_pairs ? prm.total_tiles : max_pairs;
        prm.epi_wps = tc_epi_wps(p->BN, prm.total_tiles / npairs);
        return tc_launch_wsp(mode, epi, 2 * npairs, p->wsp_smem_bytes, s, p->mapA_wsp, p->mapB_half, prm);
    }
    int TW, TH, TB;
    pick_geometry(d.Wo, d.Ho, batch, &TW, &TH, &TB);
    TcGeom* g = nullptr;
    for (int i = 0; i < p->n_geoms; i++)
        if (p->geoms[i].TW == TW && p->geoms[i].TH == TH && p->geoms[i].TB == TB) g = &p->geoms[i];
    if (!g) {
        if (p->n_geoms == 8) p->n_geoms = 0;
        g = &p->geoms[p->n_geoms];
        g->TW = TW; g->TH = TH; g->TB = TB;
        if (!encode_A(p, g)) return -1;
        p->n_geoms++;
    }
    TcParams prm = {};
    prm.t = t; prm.res = res; prm.acc_out = acc_out; prm.out = out; prm.err = d_err;
    prm.out2 = (out_bn2 && t.bn_in) ? out_bn2 : nullptr;
    prm.batch = batch; prm.Ho = d.Ho; prm.Wo = d.Wo; prm.Cout = d.Cout;
    prm.taps = d.Kh * d.Kw; prm.Kw = d.Kw; prm.Cp = d.Cin_pad; prm.cin_blocks = d.Cin_pad / p->KC;
    prm.stride = d.stride; prm.pad = d.pad;
    prm.TW = TW; prm.TH = TH; prm.TB = TB;
    prm.tiles_w = (d.Wo + TW - 1) / TW; prm.tiles_h = (d.Ho + TH - 1) / TH; prm.tiles_b = (batch + TB - 1) / TB;
    prm.tiles_n = d.Cout / p->BN;
    prm.total_tiles = prm.tiles_w * prm.tiles_h * prm.tiles_b * prm.tiles_n;
    prm.stages = p->stages; prm.group = p->group; prm.lut_bytes = p->lut_bytes; prm.ntab = p->ntab;
    prm.full_wait = TC_WAIT_CYCLES; prm.drop_stage = -1;
#ifdef FF_TC_TIMING
    prm.dbg = dbg;
#endif
    { const char* e = getenv("FF_TC_STAGES"); if (e && atoi(e) >= 2 && atoi(e) < prm.stages) prm.stages = atoi(e); }
    if (p->pair) {
        const int m_tiles = prm.tiles_w * prm.tiles_h * prm.tiles_b;
        const int pairs = prm.tiles_n * ((m_tiles + 1) / 2);
        const int max_pairs = p->n_sm / 2;
        prm.stages = p->pair_stages; prm.group = p->pair_group;
        { const char* e = getenv("FF_TC_STAGES"); if (e && atoi(e) >= 2 && atoi(e) < prm.stages) prm.stages = atoi(e); }
        int npairs = pairs < max_pairs ? pairs : max_pairs;
        if (npairs > prm.tiles_n) npairs -= npairs % prm.tiles_n;      // a pair keeps one column tile (its BN table)
        const int pgrid = 2 * npairs;
        prm.epi_wps = tc_epi_wps(p->BN, pairs / npairs);
        return tc_launch_pair(p->BN, mode, epi, p->out_f32, pgrid, p->pair_smem_bytes, s, g->mapA, p->mapB_half, prm);
    }
    int grid = prm.total_tiles < p->n_sm ? prm.total_tiles : p->n_sm;
    if (grid > prm.tiles_n) grid -= grid % prm.tiles_n;                // a CTA keeps one column tile (its BN table)
    prm.epi_wps = tc_epi_wps(p->BN, prm.total_tiles / grid);
    if (g_test_drop_stage >= 0) {                                      // armed for this one launch by the timeout test
        prm.drop_stage = g_test_drop_stage;
        if (g_test_full_wait > 0) prm.full_wait = g_test_full_wait;
        g_test_drop_stage = -1; g_test_full_wait = 0;
    }
    return tc_launch_generic(p->BN, p->KC, mode, epi, p->out_f32, grid, p->smem_bytes, s, g->mapA, p->mapB, prm);
}


// ---------------------------------------------------------------------------
// Stride-2 convolution + the block's 1x1 stride-2 shortcut in one launch (conv_tc_sc.cu)
// ---------------------------------------------------------------------------
struct ScPlan {
    TcPlan* main;            // the main path's plan for 64-column tiles (tensor maps of its input and weights)
    ffcu_layer d2;           // the shortcut layer
    const int8_t* d_in2;
    CUtensorMap mapB2;       // shortcut weights [Cout][Cin2], box {KC, 64}
    TcGeom geoms2[8];        // shortcut input boxes per tile geometry
    int n_geoms2;
    int kb_sc, stages, group, smem_bytes, lut_bytes;
};

static bool encode_A2(ScPlan* sp, TcGeom* g)
{
    encode_tiled_fn enc = get_encode();
    const ffcu_layer& d = sp->d2;
    const int KC = sp->main->KC;
    const cuuint64_t Cp = (cuuint64_t)d.Cin_pad;
    cuuint64_t dims[4] = {Cp, (cuuint64_t)d.W, (cuuint64_t)d.H, (cuuint64_t)sp->main->max_batch};
    cuuint64_t strides[3] = {Cp, Cp * d.W, Cp * d.W * d.H};
    // box of KC bytes per pixel even where the shortcut's input has fewer channels: the rest is out-of-range fill (zeros)
    cuuint32_t box[4] = {(cuuint32_t)KC, (cuuint32_t)(g->TW * 2), (cuuint32_t)(g->TH * 2), (cuuint32_t)g->TB};
    cuuint32_t estr[4] = {1, 2, 2, 1};
    if (g->TW == 1) { box[1] = 1; estr[1] = 1; }
    if (g->TH == 1) { box[2] = 1; estr[2] = 1; }
    CUresult r = enc(&g->mapA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)sp->d_in2, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, KC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(shortcut A) failed: %d", (int)r); return false; }
    return true;
}

// main: 3x3 stride-2 pad-1 convolution without residual or fused BN; sc: 1x1 stride-2 pad-0 convolution with the same
// output shape whose residual is main's output.  NULL when the pair does not fit the kernel.
ScPlan* ffcu_sc_plan(const ffcu_layer& main, const ffcu_layer& sc, int max_batch, const int8_t* d_in_main, const int8_t* d_w_main,
                     const int8_t* d_in_sc, const int8_t* d_w_sc, int device)
{
    encode_tiled_fn enc = get_encode();
    if (!enc) return nullptr;
    if (main.kind != FFCU_CONV || sc.kind != FFCU_CONV || main.Kh != 3 || main.Kw != 3 || main.stride != 2 || main.pad != 1 ||
        sc.Kh != 1 || sc.Kw != 1 || sc.stride != 2 || sc.pad != 0 || main.Cout != sc.Cout || main.Ho != sc.Ho || main.Wo != sc.Wo ||
        main.H != sc.H || main.W != sc.W || main.Cout % 64 != 0 || main.Cout > TC_MAX_COUT || sc.Cin_pad % 64 != 0)
        return nullptr;
    TcPlan* mp = ffcu_tc_plan(main, max_batch, d_in_main, d_w_main, device, 64);
    if (!mp) return nullptr;
    ScPlan* sp = new ScPlan();
    sp->main = mp; sp->d2 = sc; sp->d_in2 = d_in_sc; sp->n_geoms2 = 0;
    const int KC = mp->KC;
    sp->kb_sc = (sc.Cin_pad + KC - 1) / KC;
    sp->lut_bytes = sc.bn2_dst_buf >= 0 ? 64 * 256 : 0;
    const int sub_bytes = (TC_TILE_M + 64) * KC;
    const int fixed = 10 * TC_MAX_COUT * 4 + sp->lut_bytes + (int)sizeof(TcShared) + 1024;
    // K blocks per stage: the main plan's, or the next smaller divisor of the K loop that leaves two stages beside the
    // second table set and the byte table this kernel holds
    const int kblocks = 9 * (main.Cin_pad / KC);
    int group = mp->group, st = 0;
    for (; group >= 1; group--) {
        if (kblocks % group) continue;
        st = (232448 - fixed) / (group * sub_bytes);
        if (st >= 2) break;
    }
    if (st > TC_MAX_STAGES) st = TC_MAX_STAGES;
    if (group < 1 || st < 2 || sp->kb_sc > group || 2 * group > 32) { ffcu_tc_free(mp); delete sp; return nullptr; }
    sp->stages = st; sp->group = group;
    sp->smem_bytes = st * group * sub_bytes + fixed;
    cuuint64_t K2 = (cuuint64_t)sc.Cin_pad;
    cuuint64_t dims[4] = {K2, (cuuint64_t)sc.Cout, 1, 1};
    cuuint64_t strides[3] = {K2, K2 * sc.Cout, K2 * sc.Cout};
    cuuint32_t box[4] = {(cuuint32_t)KC, 64, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&sp->mapB2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_w_sc, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, KC == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ffcu_tc_free(mp); delete sp; cudaGetLastError(); return nullptr; }
    return sp;
}

void ffcu_sc_free(ScPlan* sp)
{
    if (!sp) return;
    ffcu_tc_free(sp->main);
    delete sp;
}

// t1 / t2: the main path's and the shortcut's tables; out_main: where the main path's int8 output goes when another
// layer reads it (write_main), out_sc / out2_sc: the block's output and its fused BN output (or NULL).
int ffcu_sc_launch(const ScPlan* csp, int batch, int mode, const EpiTables& t1, const EpiTables& t2, int8_t* out_main,
                   int write_main, int8_t* out_sc, int8_t* out2_sc, int* d_err, cudaStream_t s)
{
    ScPlan* sp = const_cast<ScPlan*>(csp);
    TcPlan* p = sp->main;
    if (batch < 1 || batch > p->max_batch) { ffcu_set_error("shortcut-fused launch: batch out of range"); return -1; }
    const ffcu_layer& d = p->d;
    int TW, TH, TB;
    pick_geometry(d.Wo, d.Ho, batch, &TW, &TH, &TB);
    TcGeom* g = nullptr;
    for (int i = 0; i < p->n_geoms; i++)
        if (p->geoms[i].TW == TW && p->geoms[i].TH == TH && p->geoms[i].TB == TB) g = &p->geoms[i];
    if (!g) {
        if (p->n_geoms == 8) p->n_geoms = 0;
        g = &p->geoms[p->n_geoms];
        g->TW = TW; g->TH = TH; g->TB = TB;
        if (!encode_A(p, g)) return -1;
        p->n_geoms++;
    }
    TcGeom* g2 = nullptr;
    for (int i = 0; i < sp->n_geoms2; i++)
        if (sp->geoms2[i].TW == TW && sp->geoms2[i].TH == TH && sp->geoms2[i].TB == TB) g2 = &sp->geoms2[i];
    if (!g2) {
        if (sp->n_geoms2 == 8) sp->n_geoms2 = 0;
        g2 = &sp->geoms2[sp->n_geoms2];
        g2->TW = TW; g2->TH = TH; g2->TB = TB;
        if (!encode_A2(sp, g2)) return -1;
        sp->n_geoms2++;
    }
    TcParams prm = {};
    prm.t = t1; prm.res = nullptr; prm.acc_out = nullptr; prm.out = out_main; prm.out2 = nullptr; prm.err = d_err;
    prm.batch = batch; prm.Ho = d.Ho; prm.Wo = d.Wo; prm.Cout = d.Cout;
    prm.taps = 9; prm.Kw = 3; prm.Cp = d.Cin_pad; prm.cin_blocks = d.Cin_pad / p->KC;
    prm.stride = 2; prm.pad = 1;
    prm.TW = TW; prm.TH = TH; prm.TB = TB;
    prm.tiles_w = (d.Wo + TW - 1) / TW; prm.tiles_h = (d.Ho + TH - 1) / TH; prm.tiles_b = (batch + TB - 1) / TB;
    prm.tiles_n = d.Cout / 64;
    prm.total_tiles = prm.tiles_w * prm.tiles_h * prm.tiles_b * prm.tiles_n;
    prm.stages = sp->stages; prm.group = sp->group; prm.lut_bytes = 0; prm.ntab = 5;
    prm.full_wait = TC_WAIT_CYCLES; prm.drop_stage = -1;
#ifdef FF_TC_TIMING
    prm.dbg = 0;
#endif
    int grid = prm.total_tiles < p->n_sm ? prm.total_tiles : p->n_sm;
    if (grid > prm.tiles_n) grid -= grid % prm.tiles_n;
    prm.epi_wps = tc_epi_wps(64, prm.total_tiles / grid);
    ScParams q = {};
    q.t2 = t2; q.out_sc = out_sc; q.out2_sc = (out2_sc && t2.bn_lut && sp->lut_bytes) ? out2_sc : nullptr;
    q.kb_sc = sp->kb_sc; q.write_main = (write_main && out_main) ? 1 : 0; q.lut_bytes = q.out2_sc ? sp->lut_bytes : 0;
    return tc_launch_sc(p->KC, mode, grid, sp->smem_bytes, s, g->mapA, p->mapB, g2->mapA, sp->mapB2, prm, q);
}

// ---------------------------------------------------------------------------
// Layer chain (conv_tc_chain.cu): plan = the first input's tensor map, the per-layer records in
// device memory (weights' tensor map, table / buffer pointers) and the shared-memory budget
// ---------------------------------------------------------------------------
struct ChainPlan {
    CUtensorMap mapA;
    ChainLayer* d_layers;
    ChainParams prm;
    int smem_bytes;
};

// layers[i]: device pointers of layer i (weights, tables, residual, outputs); all layers are 3x3 stride-1
// pad-1 convolutions C -> C on an H x W map, layer i + 1 reading what layer i writes (its fused BN's
// output where it has one).  d_in = the first layer's input (one face, NHWC).  NULL when the shape does
// not fit the kernel (C / 64 column tiles x row tiles of 128 positions must be exactly eight CTAs).
ChainPlan* ffcu_chain_plan(int H, int W, int C, const int8_t* d_in, const ChainLayerDesc* layers, int n_layers, int device)
{
    (void)device;
    encode_tiled_fn enc = get_encode();
    if (!enc || n_layers < 2 || C % 128 != 0 || C > TC_MAX_COUT) return nullptr;
    // pitch: a power of two >= W + 1.  With P = W + 1 the right-hand padding of a row is the next row's
    // left-hand slot, and the last tap of the last row reads one line past row H: one more (zero) row.
    int P = 1;
    while (P < W + 1) P <<= 1;
    const int tiles_n = C / CHAIN_BN;
    const int tiles_m = (H * P + TC_TILE_M - 1) / TC_TILE_M;
    // rows a CTA holds: the padded rows its row tile's outputs read (first output row .. last + 2)
    int rows = 0;
    for (int t = 0; t < tiles_m; t++) {
        const int olo = (t * TC_TILE_M) / P;
        int ohi = (t * TC_TILE_M + TC_TILE_M - 1) / P;
        if (ohi > H - 1) ohi = H - 1;
        if (ohi - olo + 3 > rows) rows = ohi - olo + 3;
    }
    rows += (P == W + 1 ? 1 : 0);
    if (tiles_n * tiles_m != CHAIN_CLUSTER || P > 256 || P % 8 != 0 || rows > 256) return nullptr;
    const int planes = C / 128;
    if (planes != 2 && planes != 4) return nullptr;       // the issue loops are built for 256 and 512 channels
    const int plane_bytes = P * rows * 128;
    if (plane_bytes % 1024 != 0) return nullptr;
    const int fixed = 2 * planes * plane_bytes + CHAIN_BN * 256 + 5 * CHAIN_BN * 4 + 512 /* barriers */ + 1024 /* alignment */;
    // Filter taps per stage of the weight ring (1, or 3 where two such stages fit and $FF_CHAIN_TPS=3 asks for it).
    int tps = 1;
    { const char* e = getenv("FF_CHAIN_TPS"); if (e && (atoi(e) == 1 || atoi(e) == 3) && planes == 2) tps = atoi(e); }
    while (tps > 1 && (232448 - fixed) / (tps * planes * CHAIN_BN * 128) < 2) tps /= 3;
    const int stage_bytes = tps * planes * CHAIN_BN * 128;
    int stages = (232448 - fixed) / stage_bytes;
    if (stages > CHAIN_MAX_STAGES) stages = CHAIN_MAX_STAGES;
    stages &= ~1;                                         // two issuers on alternate stages: the ring must be even
    if (stages < 2) return nullptr;
    if (!tc_chain_fits(fixed + stages * stage_bytes)) return nullptr;      // no room for a cluster of eight on this device
    ChainPlan* p = new ChainPlan();
    p->d_layers = nullptr;
    {
        cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, 1};
        cuuint64_t strides[3] = {(cuuint64_t)C, (cuuint64_t)C * W, (cuuint64_t)C * W * H};
        cuuint32_t box[4] = {128, (cuuint32_t)P, (cuuint32_t)rows, 1};
        cuuint32_t es[4] = {1, 1, 1, 1};
        CUresult r = enc(&p->mapA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_in, dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(chain A) failed: %d", (int)r); delete p; return nullptr; }
    }
    std::vector<ChainLayer> h((size_t)n_layers);
    memset(h.data(), 0, h.size() * sizeof(ChainLayer));
    for (int i = 0; i < n_layers; i++) {
        const ChainLayerDesc& d = layers[i];
        cuuint64_t Ktot = (cuuint64_t)9 * C;
        cuuint64_t dims[4] = {Ktot, (cuuint64_t)C, 1, 1};
        cuuint64_t strides[3] = {Ktot, Ktot * C, Ktot * C};
        cuuint32_t box[4] = {128, CHAIN_BN, 1, 1};
        cuuint32_t es[4] = {1, 1, 1, 1};
        CUresult r = enc(&h[i].mapB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d.w, dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(chain B) failed: %d", (int)r); delete p; return nullptr; }
        h[i].w_scale = d.t.w_scale; h[i].bias = d.t.bias; h[i].slope = d.t.slope;
        h[i].res_scale = d.res ? d.t.res_scale : nullptr; h[i].inv_out = d.t.inv_out;
        h[i].lut = (d.out2 && d.t.bn_lut) ? d.t.bn_lut : nullptr;
        h[i].res = (d.res && d.t.res_scale) ? d.res : nullptr;
        h[i].out = d.out; h[i].out2 = (d.out2 && d.t.bn_lut) ? d.out2 : nullptr;
    }
    if (cudaMalloc(&p->d_layers, h.size() * sizeof(ChainLayer)) != cudaSuccess ||
        cudaMemcpy(p->d_layers, h.data(), h.size() * sizeof(ChainLayer), cudaMemcpyHostToDevice) != cudaSuccess) {
        ffcu_set_error("layer chain: device allocation or upload failed");
        cudaFree(p->d_layers); cudaGetLastError(); delete p; return nullptr;
    }
    p->prm.layers = p->d_layers; p->prm.n_layers = n_layers;
    p->prm.H = H; p->prm.W = W; p->prm.P = P; p->prm.C = C;
    p->prm.planes = planes; p->prm.plane_bytes = plane_bytes; p->prm.win_rows = rows; p->prm.tiles_n = tiles_n; p->prm.stages = stages; p->prm.tps = tps;
    p->prm.err = nullptr;
    p->smem_bytes = fixed + stages * stage_bytes;
    return p;
}

void ffcu_chain_free(ChainPlan* p)
{
    if (!p) return;
    cudaFree(p->d_layers);
    delete p;
}

// One-shot fault injection for the layer chain's timeout-path test: consumed by the next chain launch.
static int g_test_chain_drop_step = -1;
static long long g_test_chain_wait = 0;

extern "C" void ffcu_test_arm_chain_timeout(int drop_step, long long wait_cycles)
{
    g_test_chain_drop_step = drop_step;
    g_test_chain_wait = wait_cycles;
}

int ffcu_chain_launch(const ChainPlan* p, int mode, int* d_err, cudaStream_t s)
{
    ChainParams prm = p->prm;
    prm.err = d_err;
    prm.wait_cycles = TC_WAIT_CYCLES; prm.drop_step = -1;
    if (g_test_chain_drop_step >= 0) {                    // armed for this one launch
        prm.drop_step = g_test_chain_drop_step;
        if (g_test_chain_wait > 0) prm.wait_cycles = g_test_chain_wait;
        g_test_chain_drop_step = -1; g_test_chain_wait = 0;
    }
#ifdef FF_TC_TIMING
    // timing build, $FF_CHAIN_TS=1: the 30th launch of a chain prints CTA 0's per-layer time stamps
    { static int dbg = -1; if (dbg < 0) { const char* e = getenv("FF_TC_DBG"); dbg = e ? atoi(e) : 0; } prm.dbg = dbg; }
    static unsigned long long* d_ts = nullptr;
    static int calls = 0;
    prm.ts = nullptr;
    if (getenv("FF_CHAIN_TS")) {
        if (!d_ts) cudaMalloc(&d_ts, 64 * 4 * sizeof(unsigned long long));
        prm.ts = d_ts;
        if (++calls == 29 || calls == 30) {
            int rc = tc_launch_chain(mode, p->smem_bytes, s, p->mapA, prm);
            cudaStreamSynchronize(s);
            unsigned long long h[256];
            cudaMemcpy(h, d_ts, sizeof h, cudaMemcpyDeviceToHost);
            for (int L = 0; L < prm.n_layers; L++)
                fprintf(stderr, "chain L%d: in->mma_issued %lld, mma_issued->acc %lld, acc->sent %lld, sent->next_in %lld ns\n", L,
                        (long long)(h[4 * L + 1] - h[4 * L]), (long long)(h[4 * L + 2] - h[4 * L + 1]), (long long)(h[4 * L + 3] - h[4 * L + 2]),
                        L + 1 < prm.n_layers ? (long long)(h[4 * L + 4] - h[4 * L + 3]) : 0ll);
            return rc;
        }
    }
#endif
    return tc_launch_chain(mode, p->smem_bytes, s, p->mapA, prm);
}

// ---------------------------------------------------------------------------
// Tensor-core stem (conv_tc_stem.cu): plan = the weights' tensor map and the launch geometry
// ---------------------------------------------------------------------------
struct StemTcPlan {
    CUtensorMap mapB;
    int max_batch, n_sm, stages, smem_bytes, lut_bytes;
};

StemTcPlan* ffcu_stem_tc_plan(int max_batch, const int8_t* d_wk, bool has_bn2, int device)
{
    encode_tiled_fn enc = get_encode();
    if (!enc) { ffcu_set_error("cuTensorMapEncodeTiled is not available"); return nullptr; }
    StemTcPlan* p = new StemTcPlan();
    p->max_batch = max_batch;
    cudaDeviceGetAttribute(&p->n_sm, cudaDevAttrMultiProcessorCount, device);
    cuuint32_t es[4] = {1, 1, 1, 1};
    cuuint64_t bdims[4] = {32, 64, 1, 1};
    cuuint64_t bstr[3] = {32, 32 * 64, 32 * 64};
    cuuint32_t bbox[4] = {32, 64, 1, 1};
    CUresult r = enc(&p->mapB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)d_wk, bdims, bstr, bbox, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ffcu_set_error("cuTensorMapEncodeTiled(stem) failed: %d", (int)r); delete p; return nullptr; }
    p->lut_bytes = has_bn2 ? 64 * 256 : 0;
    p->stages = TC_MAX_STAGES;                             // even: two producer warps take alternate tiles
    p->smem_bytes = 64 * 32 + p->stages * TC_TILE_M * 32 + 5 * TC_MAX_COUT * 4 + p->lut_bytes + (int)sizeof(TcShared) + 2048;
    return p;
}

void ffcu_stem_tc_free(StemTcPlan* p) { delete p; }

// One-launch stem (conv_tc_stem.cu): the producers read the network input themselves.
int ffcu_stem_fused_launch(const StemTcPlan* p, const void* in_any, int in_u8, const float* inv3, int batch, int mode,
                           const EpiTables& t, int8_t* out, int8_t* out_bn2, int* d_err, cudaStream_t s)
{
    if (batch < 1 || batch > p->max_batch) { ffcu_set_error("stem launch: batch out of range"); return -1; }
    const bool has_slope = t.slope != nullptr, has_bn2 = out_bn2 && t.bn_in && t.bn_lut && p->lut_bytes;
    int epi = EPI_RUNTIME;
    if (has_slope && has_bn2) epi = EPI_SLOPE_BN;
    else if (has_slope && !out_bn2) epi = EPI_SLOPE;
    if (!t.no_overflow || !t.acc22) epi = EPI_RUNTIME;
    TcParams prm = {};
    prm.t = t; prm.res = nullptr; prm.acc_out = nullptr; prm.out = out; prm.err = d_err;
    prm.out2 = has_bn2 ? out_bn2 : nullptr;
    prm.batch = batch; prm.Ho = 112; prm.Wo = 112; prm.Cout = 64;
    prm.taps = 1; prm.Kw = 1; prm.Cp = 32; prm.cin_blocks = 1; prm.stride = 1; prm.pad = 0;
    prm.TW = 16; prm.TH = 8; prm.TB = 1;
    prm.tiles_w = 112 / 16; prm.tiles_h = 112 / 8; prm.tiles_b = batch; prm.tiles_n = 1;
    prm.total_tiles = prm.tiles_w * prm.tiles_h * batch;
    prm.stages = p->stages; prm.group = 1; prm.lut_bytes = has_bn2 ? p->lut_bytes : 0; prm.ntab = 5;
    prm.full_wait = TC_WAIT_CYCLES; prm.drop_stage = -1;
#ifdef FF_TC_TIMING
    { static int dbg = -1; if (dbg < 0) { const char* e = getenv("FF_TC_DBG"); dbg = e ? atoi(e) : 0; } prm.dbg = dbg; }
#endif
    const int grid = prm.total_tiles < p->n_sm ? prm.total_tiles : p->n_sm;
    prm.epi_wps = tc_epi_wps(64, prm.total_tiles / grid);
    return tc_launch_stem(mode, epi, in_u8, grid, p->smem_bytes, s, p->mapB, prm, in_any, inv3);
}
