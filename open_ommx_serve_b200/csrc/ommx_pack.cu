// KV quantize + pack ("store") kernels for sm_100a.
//
// Replaces ommx_pack_kv_canonical_block (ommx_gpu_serve/attention/pack.py:293-655 of the
// reference) and writes straight into destination pages / group slots.  Output planes are
// bit-identical to the reference packer run on CPU: every arithmetic step is the same IEEE
// fp32 operation in the same order (no FMA contraction: explicit __f*_rn intrinsics), and the
// two library calls of the reference (log2, log) are replaced by frozen threshold tables.
//
// K kernel: one warp per (32-token group, kv head, 16-channel block); lane = token.  Outlier
//   selection is the reference's stable-sort rule done with warp reductions: the r-th pick is the
//   max (min) key over unpicked lanes, ties to the lowest lane (redux.sync + ballot).
// V kernel: one thread per (token, head, 32-channel group).
#include "ommx_common.cuh"

namespace ommx {

__constant__ uint32_t c_pow2_cut[256] = {OMMX_POW2_CUT_VALUES};
__constant__ uint32_t c_fp4_thresh[7] = {OMMX_FP4_THRESH_VALUES};

template <typename T> __device__ __forceinline__ float load_as_f32(const T *p);
template <> __device__ __forceinline__ float load_as_f32<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __bfloat162float(*p);
}
template <> __device__ __forceinline__ float load_as_f32<__half>(const __half *p) { return __half2float(*p); }

// Monotone map fp32 -> uint32 (larger float <=> larger key); -0.0 is folded onto +0.0 first so
// that equal values tie exactly as they do under the reference's float comparisons.
__device__ __forceinline__ uint32_t f32_key(float x) {
    uint32_t u = __float_as_uint(x + 0.0f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_f32(uint32_t k) {
    uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
    return __uint_as_float(u);
}

struct PackKParams {
    const void *k;
    int64_t stride_token, stride_head;
    int32_t num_groups, H, D, page_size;
    const int32_t *dst_pages, *dst_groups;
    int32_t num_pages, num_group_slots;
    int32_t k_out, select_signed, use_pow2, outlier_map, scale_kind;
    uint8_t *k_base;
    void *k_scale, *k_zp, *k_mapscale, *k_mapcenter;
    uint8_t *k_obmp, *k_oval;
    int32_t *status;
};

constexpr int PACK_WARPS = 4;
constexpr int PACK_BLK = 16;                       // channels per warp: one 32-bit word of 2-bit codes per token

// scale -> (value after optional pow2 snap and storage rounding, exponent)
__device__ __forceinline__ float snap_scale(float rng, int use_pow2, int scale_kind, int &e) {
    float scale = __fdiv_rn(fmaxf(rng, 1e-8f), 3.0f);
    e = 0;
    if (use_pow2) {
        e = pow2_exponent_tbl(fmaxf(scale, 1e-12f), c_pow2_cut);
        scale = __uint_as_float((uint32_t)(e + 127) << 23);
    }
    if (scale_kind != OMMX_SCALE_F32) scale = bf16_round_f32(scale);
    return scale;
}

// One warp per (32-token group, kv head, block of 16 channels); lane = token.  A lane reads its 16
// channel values straight from global memory; the 16 two-bit codes of the block are exactly one
// 32-bit word of the token's row, so warps never share an output word.
template <typename T>
__global__ void __launch_bounds__(PACK_WARPS * 32) pack_k_kernel(PackKParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = p.D / PACK_BLK;
    const int unit = blockIdx.x * PACK_WARPS + warp;           // (group, head, channel block)
    if (unit >= p.num_groups * p.H * nblk) return;
    const int blk = unit % nblk;
    const int gh = unit / nblk;
    const int g = gh / p.H, h = gh - g * p.H;
    const int D = p.D;

    const T *row = reinterpret_cast<const T *>(p.k) + (int64_t)(g * 32 + lane) * p.stride_token
                 + (int64_t)h * p.stride_head + blk * PACK_BLK;
    float xv[PACK_BLK];
#pragma unroll
    for (int c = 0; c < PACK_BLK; ++c) xv[c] = load_as_f32(row + c);

    // destination addressing
    const int ps = p.page_size;
    const int tok = g * 32 + lane;
    int page = tok / ps;
    if (p.dst_pages) page = p.dst_pages[page];
    int slot = p.dst_groups ? p.dst_groups[g] : g;
    bool page_ok = (page >= 0 && page < p.num_pages);
    bool slot_ok = (slot >= 0 && slot < p.num_group_slots);
    if (!page_ok) or_status(p.status, OMMX_ST_BAD_PAGE);
    if (!slot_ok && lane == 0) or_status(p.status, OMMX_ST_BAD_GROUP);

    const int k = p.k_out;
    const int kt = p.select_signed ? (k + 1) / 2 : k;
    const int kb = p.select_signed ? k - kt : 0;
    const int nb = (k + 1) / 2;
    const uint32_t lt_mask = (1u << lane) - 1u;
    const bool store_f32 = (p.scale_kind == OMMX_SCALE_F32);
    const int64_t gbase = ((int64_t)slot * p.H + h) * D + blk * PACK_BLK;   // element offset in [G,H,D] planes

    uint32_t word = 0;
    bool bad = false;
    // per-channel parameters, parked on lane cc (lanes 0..15)
    int my_e = 0;
    float my_scale = 0.f, my_zp = 0.f, my_ms = 0.f, my_mc = 0.f;
    uint32_t my_bmp = 0;
    unsigned long long my_val = 0ull;

#pragma unroll
    for (int cc = 0; cc < PACK_BLK; ++cc) {
        const float x = xv[cc];
        if (!isfinite(x)) bad = true;
        const uint32_t key = p.select_signed ? f32_key(x) : (__float_as_uint(fabsf(x)) + 1u);
        // ---- outlier selection: r-th pick = extreme key over unpicked lanes, ties -> lowest lane ----
        bool sel = false;
        for (int r = 0; r < kt; ++r) {
            uint32_t cand = sel ? 0u : key;
            uint32_t m = __reduce_max_sync(0xFFFFFFFFu, cand);
            uint32_t hit = __ballot_sync(0xFFFFFFFFu, !sel && cand == m);
            if (hit && lane == (__ffs(hit) - 1)) sel = true;
        }
        for (int r = 0; r < kb; ++r) {
            uint32_t cand = sel ? 0xFFFFFFFFu : key;
            uint32_t m = __reduce_min_sync(0xFFFFFFFFu, cand);
            uint32_t hit = __ballot_sync(0xFFFFFFFFu, !sel && cand == m);
            if (hit && lane == (__ffs(hit) - 1)) sel = true;
        }
        const uint32_t omask = __ballot_sync(0xFFFFFFFFu, sel);
        // ---- base affine over the non-outlier lanes ----
        const uint32_t vkey = f32_key(x);
        uint32_t kmin = __reduce_min_sync(0xFFFFFFFFu, sel ? 0xFFFFFFFFu : vkey);
        uint32_t kmax = __reduce_max_sync(0xFFFFFFFFu, sel ? 0u : vkey);
        float mn = (omask == 0xFFFFFFFFu) ? 0.f : key_f32(kmin);
        float mx = (omask == 0xFFFFFFFFu) ? 0.f : key_f32(kmax);
        int e;
        const float scale = snap_scale(__fsub_rn(mx, mn), p.use_pow2, p.scale_kind, e);
        const float zp = store_f32 ? mn : bf16_round_f32(mn);
        float qv = rintf(__fdiv_rn(__fsub_rn(x, zp), scale));
        qv = fminf(fmaxf(qv, 0.f), 3.f);
        word |= (uint32_t)(int)qv << (2 * cc);
        // ---- outlier values ----
        float ms = 0.f, mc = 0.f;
        unsigned long long val = 0ull;
        if (k > 0) {
            float mapped;
            if (p.outlier_map) {
                uint32_t okmin = __reduce_min_sync(0xFFFFFFFFu, sel ? vkey : 0xFFFFFFFFu);
                uint32_t okmax = __reduce_max_sync(0xFFFFFFFFu, sel ? vkey : 0u);
                float omn = key_f32(okmin), omx = key_f32(okmax);
                mc = __fmul_rn(__fadd_rn(omx, omn), 0.5f);
                // the reference evaluates 12.0 / range as reciprocal(range) * 12
                ms = __fmul_rn(__frcp_rn(fmaxf(__fsub_rn(omx, omn), 1e-8f)), 12.0f);
                if (!store_f32) { mc = bf16_round_f32(mc); ms = bf16_round_f32(ms); }
                mapped = __fmul_rn(__fsub_rn(x, mc), ms);
            } else {
                mapped = __fdiv_rn(__fsub_rn(x, zp), scale);
            }
            uint32_t fp4 = (uint32_t)fp4_encode_tbl(mapped, c_fp4_thresh);
            int rank = __popc(omask & lt_mask);
            unsigned long long contrib = (sel && rank < 16) ? ((unsigned long long)fp4 << (4 * rank)) : 0ull;
            uint32_t lo = __reduce_or_sync(0xFFFFFFFFu, (uint32_t)contrib);
            uint32_t hi = (k > 8) ? __reduce_or_sync(0xFFFFFFFFu, (uint32_t)(contrib >> 32)) : 0u;
            val = ((unsigned long long)hi << 32) | lo;
        }
        if (lane == cc) {
            my_e = e; my_scale = scale; my_zp = zp; my_ms = ms; my_mc = mc; my_bmp = omask; my_val = val;
        }
    }
    // ---- lanes 0..15 write the block's 16 consecutive channel entries ----
    if (slot_ok && lane < PACK_BLK) {
        const int64_t off = gbase + lane;
        if (p.scale_kind == OMMX_SCALE_INT8_EXP) reinterpret_cast<int8_t *>(p.k_scale)[off] = (int8_t)my_e;
        else if (p.scale_kind == OMMX_SCALE_BF16) reinterpret_cast<uint16_t *>(p.k_scale)[off] = (uint16_t)f32_to_bf16_bits(my_scale);
        else reinterpret_cast<float *>(p.k_scale)[off] = my_scale;
        if (store_f32) reinterpret_cast<float *>(p.k_zp)[off] = my_zp;
        else reinterpret_cast<uint16_t *>(p.k_zp)[off] = (uint16_t)f32_to_bf16_bits(my_zp);
        if (k > 0) {
            if (p.outlier_map) {
                if (store_f32) {
                    reinterpret_cast<float *>(p.k_mapscale)[off] = my_ms;
                    reinterpret_cast<float *>(p.k_mapcenter)[off] = my_mc;
                } else {
                    reinterpret_cast<uint16_t *>(p.k_mapscale)[off] = (uint16_t)f32_to_bf16_bits(my_ms);
                    reinterpret_cast<uint16_t *>(p.k_mapcenter)[off] = (uint16_t)f32_to_bf16_bits(my_mc);
                }
            }
            reinterpret_cast<uint32_t *>(p.k_obmp)[off] = my_bmp;
            for (int i = 0; i < nb; ++i) p.k_oval[off * nb + i] = (uint8_t)(my_val >> (8 * i));
        }
    }
    if (bad) or_status(p.status, OMMX_ST_NONFINITE);
    if (page_ok) {
        uint8_t *dst = p.k_base + (((int64_t)page * ps + (tok % ps)) * p.H + h) * (D / 4);
        reinterpret_cast<uint32_t *>(dst)[blk] = word;
    }
}

struct PackVParams {
    const void *v;
    int64_t stride_token, stride_head;
    int32_t num_tokens, H, D, page_size;
    const int32_t *dst_pages;
    int32_t num_pages, use_pow2, scale_kind;
    uint8_t *v_main;
    void *v_scale, *v_zp;
    int32_t *status;
};

template <typename T>
__global__ void __launch_bounds__(128) pack_v_kernel(PackVParams p) {
    const int ngv = p.D / 32;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)p.num_tokens * p.H * ngv) return;
    const int cg = (int)(idx % ngv);
    const int h = (int)((idx / ngv) % p.H);
    const int t = (int)(idx / ((int64_t)ngv * p.H));
    const T *row = reinterpret_cast<const T *>(p.v) + (int64_t)t * p.stride_token + (int64_t)h * p.stride_head + cg * 32;
    float x[32];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        x[i] = load_as_f32(row + i);
        if (!isfinite(x[i])) bad = true;
    }
    float mn = x[0], mx = x[0];
#pragma unroll
    for (int i = 1; i < 32; ++i) { mn = fminf(mn, x[i]); mx = fmaxf(mx, x[i]); }
    mn += 0.0f;
    int e;
    const float scale = snap_scale(__fsub_rn(mx, mn), p.use_pow2, p.scale_kind, e);
    const bool store_f32 = (p.scale_kind == OMMX_SCALE_F32);
    const float zp = store_f32 ? mn : bf16_round_f32(mn);
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float qv = rintf(__fdiv_rn(__fsub_rn(x[i], zp), scale));
        qv = fminf(fmaxf(qv, 0.f), 3.f);
        uint32_t c = (uint32_t)(int)qv;
        if (i < 16) w0 |= c << (2 * i); else w1 |= c << (2 * (i - 16));
    }
    if (bad) or_status(p.status, OMMX_ST_NONFINITE);
    int page = t / p.page_size;
    if (p.dst_pages) page = p.dst_pages[page];
    if (page < 0 || page >= p.num_pages) { or_status(p.status, OMMX_ST_BAD_PAGE); return; }
    const int64_t loc = ((int64_t)page * p.page_size + (t % p.page_size)) * p.H + h;
    uint2 *dst = reinterpret_cast<uint2 *>(p.v_main + loc * (p.D / 4) + cg * 8);
    *dst = make_uint2(w0, w1);
    const int64_t soff = loc * ngv + cg;
    if (p.scale_kind == OMMX_SCALE_INT8_EXP) reinterpret_cast<int8_t *>(p.v_scale)[soff] = (int8_t)e;
    else if (p.scale_kind == OMMX_SCALE_BF16) reinterpret_cast<uint16_t *>(p.v_scale)[soff] = (uint16_t)f32_to_bf16_bits(scale);
    else reinterpret_cast<float *>(p.v_scale)[soff] = scale;
    if (store_f32) reinterpret_cast<float *>(p.v_zp)[soff] = zp;
    else reinterpret_cast<uint16_t *>(p.v_zp)[soff] = (uint16_t)f32_to_bf16_bits(zp);
}

template <typename T>
static int launch_pack(const ommx_pack_args *a, cudaStream_t st) {
    const ommx_kv_planes &pl = a->planes;
    PackKParams kp;
    kp.k = a->k; kp.stride_token = a->stride_token; kp.stride_head = a->stride_head;
    kp.num_groups = a->num_tokens / 32; kp.H = pl.n_kv_heads; kp.D = pl.head_dim; kp.page_size = pl.page_size;
    kp.dst_pages = a->dst_pages; kp.dst_groups = a->dst_groups;
    kp.num_pages = pl.num_pages; kp.num_group_slots = pl.num_group_slots;
    kp.k_out = pl.outliers_per_vector; kp.select_signed = a->outlier_select; kp.use_pow2 = a->use_pow2;
    kp.outlier_map = pl.kv_outlier_map; kp.scale_kind = pl.scale_kind;
    kp.k_base = (uint8_t *)pl.k_base; kp.k_scale = pl.k_scale; kp.k_zp = pl.k_zp;
    kp.k_mapscale = pl.k_mapscale; kp.k_mapcenter = pl.k_mapcenter;
    kp.k_obmp = (uint8_t *)pl.k_obmp; kp.k_oval = (uint8_t *)pl.k_oval; kp.status = a->status;
    const int units = kp.num_groups * kp.H * (kp.D / PACK_BLK);
    if (units > 0) {
        pack_k_kernel<T><<<(units + PACK_WARPS - 1) / PACK_WARPS, PACK_WARPS * 32, 0, st>>>(kp);
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    PackVParams vp;
    vp.v = a->v; vp.stride_token = a->stride_token; vp.stride_head = a->stride_head;
    vp.num_tokens = a->num_tokens; vp.H = pl.n_kv_heads; vp.D = pl.head_dim; vp.page_size = pl.page_size;
    vp.dst_pages = a->dst_pages; vp.num_pages = pl.num_pages; vp.use_pow2 = a->use_pow2; vp.scale_kind = pl.scale_kind;
    vp.v_main = (uint8_t *)pl.v_main; vp.v_scale = pl.v_scale; vp.v_zp = pl.v_zp; vp.status = a->status;
    const int64_t nthreads = (int64_t)a->num_tokens * pl.n_kv_heads * (pl.head_dim / 32);
    if (nthreads > 0) {
        pack_v_kernel<T><<<(unsigned)((nthreads + 127) / 128), 128, 0, st>>>(vp);
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    return 0;
}

}  // namespace ommx

extern "C" int ommx_b200_pack_kv(const ommx_pack_args *a, void *stream) {
    using namespace ommx;
    if (!a) return fail(OMMX_E_ARG, "pack: null args");
    const ommx_kv_planes &pl = a->planes;
    if (!a->k || !a->v) return fail(OMMX_E_ARG, "pack: null k/v");
    if (a->num_tokens < 0 || a->num_tokens % 32 != 0)
        return fail(OMMX_E_ARG, "pack: num_tokens=%d must be a multiple of 32", a->num_tokens);
    if (pl.page_size <= 0 || 32 % pl.page_size != 0 && pl.page_size % 32 != 0)
        return fail(OMMX_E_ARG, "pack: page_size=%d must divide 32 or be a multiple of it", pl.page_size);
    if (a->num_tokens % pl.page_size != 0)
        return fail(OMMX_E_ARG, "pack: num_tokens=%d must be a multiple of page_size=%d", a->num_tokens, pl.page_size);
    if (pl.head_dim % 32 != 0 || pl.head_dim <= 0)
        return fail(OMMX_E_UNSUPPORTED, "pack: head_dim=%d must be a positive multiple of 32", pl.head_dim);
    if (pl.n_kv_heads <= 0) return fail(OMMX_E_ARG, "pack: n_kv_heads=%d", pl.n_kv_heads);
    if (pl.outliers_per_vector < 0 || pl.outliers_per_vector > 16)
        return fail(OMMX_E_UNSUPPORTED, "pack: outliers_per_vector=%d outside [0,16]", pl.outliers_per_vector);
    if (pl.scale_kind == OMMX_SCALE_INT8_EXP && !a->use_pow2)
        return fail(OMMX_E_ARG, "pack: int8 exponent scales need use_pow2");
    if (pl.scale_kind < 0 || pl.scale_kind > 2) return fail(OMMX_E_ARG, "pack: scale_kind=%d", pl.scale_kind);
    if (!pl.k_base || !pl.k_scale || !pl.k_zp || !pl.v_main || !pl.v_scale || !pl.v_zp)
        return fail(OMMX_E_ARG, "pack: a destination plane is null");
    if (pl.outliers_per_vector > 0 && (!pl.k_obmp || !pl.k_oval))
        return fail(OMMX_E_ARG, "pack: k>0 needs k_obmp and k_oval");
    if (pl.outliers_per_vector > 0 && pl.kv_outlier_map && (!pl.k_mapscale || !pl.k_mapcenter))
        return fail(OMMX_E_ARG, "pack: kv_outlier_map needs k_mapscale and k_mapcenter");
    if (((uintptr_t)pl.k_base & 3) || ((uintptr_t)pl.v_main & 7) || ((uintptr_t)pl.k_obmp & 3))
        return fail(OMMX_E_ARG, "pack: k_base/k_obmp must be 4-byte and v_main 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    switch (a->in_dtype) {
        case OMMX_DT_F32: return launch_pack<float>(a, st);
        case OMMX_DT_BF16: return launch_pack<__nv_bfloat16>(a, st);
        case OMMX_DT_F16: return launch_pack<__half>(a, st);
        default: return fail(OMMX_E_ARG, "pack: in_dtype=%d", a->in_dtype);
    }
}
