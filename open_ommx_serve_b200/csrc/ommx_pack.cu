// KV quantize + pack ("store") kernels for sm_100a.
//
// Replaces ommx_pack_kv_canonical_block (ommx_gpu_serve/attention/pack.py:293-655 of the
// reference) and writes straight into destination pages / group slots.  Output planes are
// bit-identical to the reference packer run on CPU: every arithmetic step is the same IEEE
// fp32 operation in the same order (no FMA contraction: explicit __f*_rn intrinsics), and the
// two library calls of the reference (log2, log) are replaced by frozen threshold tables.
//
// K kernels: the reference's stable-sort selection rule (the r-th pick is the max (min) key over
//   unpicked tokens, ties to the lowest token) in two interchangeable forms.  pack_k_lane_kernel
//   (signed rule, k in {0,2,4,6,8}): one warp per (group, kv head, 32 channels), lane = channel,
//   per-lane loops over 32 register values.  pack_k_kernel (any rule, k <= 16): one warp per
//   (group, kv head, 16 channels), lane = token, warp reductions (redux.sync + ballot).
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

// a 16-bit storage pattern of T as fp32 (T = float never takes this path)
template <typename T> __device__ __forceinline__ float bits16_as_f32(uint32_t b) { return 0.f; }
template <> __device__ __forceinline__ float bits16_as_f32<__nv_bfloat16>(uint32_t b) { return __uint_as_float(b << 16); }
template <> __device__ __forceinline__ float bits16_as_f32<__half>(uint32_t b) { return __half2float(__ushort_as_half((unsigned short)b)); }

// clamp(rint(x), 0, 3) as an integer without the conversion pipe: rint is monotone, so the clamp may come
// first; adding 1.5 * 2^23 then rounds to nearest-even into the low mantissa bits (exact for |x| <= 3).
__device__ __forceinline__ uint32_t code_0_3(float x) {
    const float c = fminf(fmaxf(x, 0.f), 3.f);                  // NaN -> 0
    return __float_as_uint(__fadd_rn(c, 12582912.f)) - 0x4B400000u;
}

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

// Decode-step source: instead of a linear block of tokens, unit "group" i is batch row i of a pool of
// sequences; its 32 tokens are the group the step completed (none: the unit returns), read from the
// residual ring, and its destination comes from the sequence's own page / group-slot tables.
struct PoolSrc {
    const int32_t *seq;               // null = linear source
    const void *slots;                // batch row -> sequence slot (int32 or int64), null = identity
    const void *wpos;                 // batch row -> absolute write position, null = the slot's seq entry
    const int32_t *r2t, *r2g;
    int32_t ring_cap, sink, recent, groups_per_seq, pages_per_seq;
    int32_t num_seqs, pages_per_group, idx64;
};
__device__ __forceinline__ int pool_index(const void *tbl, int is64, int i) {
    return is64 ? (int) reinterpret_cast<const int64_t *>(tbl)[i] : reinterpret_cast<const int32_t *>(tbl)[i];
}
__device__ __forceinline__ int pool_slot(const PoolSrc &ps, int i) { return ps.slots ? pool_index(ps.slots, ps.idx64, i) : i; }
// tokens the sequence of batch row i holds before this step (its write position)
__device__ __forceinline__ int pool_pos(const PoolSrc &ps, int i, int slot) {
    return ps.wpos ? pool_index(ps.wpos, ps.idx64, i) : ps.seq[slot];
}
__device__ __forceinline__ int pool_groups_at(const PoolSrc &ps, int seq) {
    const int spare = seq - ps.sink - ps.recent;
    return spare > 0 ? spare / 32 : 0;
}
// A sequence slot outside the pool, or a step that would complete a group the sequence's table rows
// cannot hold (it was stepped past its capacity): such a row is refused - nothing is written for it
// and its length does not advance - because its group would land in the NEXT sequence's pages.
__device__ __forceinline__ bool pool_row_refused(const PoolSrc &ps, int seq_slot, int pos_after) {
    if (seq_slot < 0 || seq_slot >= ps.num_seqs) return true;
    const int groups = pool_groups_at(ps, pos_after);
    return groups > ps.groups_per_seq || groups * ps.pages_per_group > ps.pages_per_seq;
}

struct PackKParams {
    PoolSrc pool;
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

// ---------------------------------------------------------------------------------------------
// K kernel, lane-per-channel form, for the signed selection rule with a compile-time (KT, KB) =
// (picks from the top, picks from the bottom).  One warp per (32-token group, kv head, 32-channel
// block); lane = channel; the lane holds its channel's 32 token values in registers, so selection,
// min/max and quantization are plain per-lane loops over registers: no warp reductions, and every
// per-channel step (scale snap, zero-point, FP4 map) runs for 32 channels at once.  The 2-bit codes
// (lane-major: one lane, 32 tokens) are turned token-major (one lane, 32 channels = the 8 bytes of
// a token's row) by a five-stage shuffle butterfly.  Same arithmetic, in the same order, as
// pack_k_kernel; the two are interchangeable bit for bit.
// ---------------------------------------------------------------------------------------------
template <typename T, int KT, int KB>
__global__ void __launch_bounds__(PACK_WARPS * 32) pack_k_lane_kernel(PackKParams p) {
    constexpr int K = KT + KB;
    constexpr int NB = (K + 1) / 2;
    static_assert(K <= 8, "the nibble stream is kept in 32 bits");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = p.D / 32;
    const int unit = blockIdx.x * PACK_WARPS + warp;           // (group, head, 32-channel block)
    if (unit >= p.num_groups * p.H * nblk) return;
    const int blk = unit % nblk;
    const int gh = unit / nblk;
    const int g = gh / p.H, h = gh - g * p.H;
    const int D = p.D;

    // ---- this channel's 32 token values ----
    const T *col = reinterpret_cast<const T *>(p.k) + (int64_t)h * p.stride_head + blk * 32 + lane;
    float x[32];
    int grp = g, seq_slot = 0;                // pool source: group index inside the sequence, sequence slot
    if (p.pool.seq) {
        seq_slot = pool_slot(p.pool, g);
        if (seq_slot < 0 || seq_slot >= p.pool.num_seqs) return;     // reported by the ring-write kernel
        const int pos = pool_pos(p.pool, g, seq_slot);
        grp = pool_groups_at(p.pool, pos);
        if (pool_groups_at(p.pool, pos + 1) == grp) return;          // this step completes no group
        if (pool_row_refused(p.pool, seq_slot, pos + 1)) { if (lane == 0) or_status(p.status, OMMX_ST_BAD_LENGTH); return; }
        const int rec = p.pool.ring_cap - p.pool.sink;
        const int first = (grp * 32) % rec;                           // ring row (behind the sink rows) of token 0
        col += (int64_t)(seq_slot * p.pool.ring_cap + p.pool.sink) * p.stride_token;
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            int rr = first + t;
            if (rr >= rec) rr -= rec;
            x[t] = load_as_f32(col + (int64_t)rr * p.stride_token);
        }
    } else {
        col += (int64_t)(g * 32) * p.stride_token;
#pragma unroll
        for (int t = 0; t < 32; ++t) x[t] = load_as_f32(col + (int64_t)t * p.stride_token);
    }

    const int slot = p.pool.seq ? p.pool.r2g[seq_slot * p.pool.groups_per_seq + grp] : (p.dst_groups ? p.dst_groups[g] : g);
    const bool slot_ok = (slot >= 0 && slot < p.num_group_slots);
    if (!slot_ok && lane == 0) or_status(p.status, OMMX_ST_BAD_GROUP);
    const bool store_f32 = (p.scale_kind == OMMX_SCALE_F32);

    bool bad = false;
    uint32_t omask = 0;
    uint32_t pick_key[K > 0 ? K : 1];
    int pick_tok[K > 0 ? K : 1];
    uint32_t kmax = 0u, kmin = 0u;
    bool rounds = true;                       // take the selection rounds below
    if constexpr (sizeof(T) == 2) {
        // One pass.  A value that came from 16 bits leaves the low 13 bits of its order key the same for every
        // token of a sign, so the token number can ride there: (key | 31 - t) orders tokens for the picks from the
        // top, (key | t) for the picks from the bottom, both with ties going to the lowest token, and all 32
        // composites differ.  Sorted insertion keeps the KT + 1 largest and the KB + 1 smallest; the entries
        // behind the picks are the extremes of what was not picked.  When a token is picked from both ends (a
        // group with fewer than K + 1 distinct values) the rule "bottom picks skip the top picks" matters, and the
        // warp takes the rounds.
        uint32_t top[KT + 1], bot[KB + 1];
#pragma unroll
        for (int i = 0; i <= KT; ++i) top[i] = 0u;
#pragma unroll
        for (int i = 0; i <= KB; ++i) bot[i] = 0xFFFFFFFFu;
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            // order key of x + 0 (the sign bit set for x >= 0, all bits flipped below), low five bits cleared
            const uint32_t u = __float_as_uint(x[t] + 0.0f);
            const uint32_t key = (u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u)) & ~31u;
            uint32_t c = key | (uint32_t)(31 - t);
#pragma unroll
            for (int i = 0; i <= KT; ++i) { const uint32_t hi = max(top[i], c); c = min(top[i], c); top[i] = hi; }
            c = key | (uint32_t)t;
#pragma unroll
            for (int i = 0; i <= KB; ++i) { const uint32_t lo = min(bot[i], c); c = max(bot[i], c); bot[i] = lo; }
        }
        // the key's own low bits: ones below zero, zeros from zero up
        auto full_key = [](uint32_t comp) { return (comp & ~31u) | ((comp & 0x80000000u) ? 0u : 31u); };
#pragma unroll
        for (int r = 0; r < K; ++r) {
            const uint32_t comp = r < KT ? top[r < KT ? r : 0] : bot[r < KT ? 0 : r - KT];
            pick_tok[r] = r < KT ? 31 - (int)(comp & 31u) : (int)(comp & 31u);
            pick_key[r] = full_key(comp);
            omask |= 1u << pick_tok[r];
        }
        kmax = full_key(top[KT]);
        kmin = full_key(bot[KB]);
        // an infinity or a NaN is the largest (smallest) key of its sign: the two ends of the order tell
        bad = top[0] >= 0xFF800000u || bot[0] < 0x00800000u;
        rounds = __any_sync(0xFFFFFFFFu, __popc(omask) != K || bad);
    }
    if (rounds) {
        uint32_t cand[32];                    // order keys; 0 marks a picked token (no finite value has key 0)
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            bad |= !isfinite(x[t]);
            cand[t] = f32_key(x[t]);
        }
        // ---- outlier selection: r-th pick = extreme key over unpicked tokens, ties -> lowest token ----
        omask = 0;
#pragma unroll
        for (int r = 0; r < K; ++r) {
            uint32_t m;
            if (r < KT) {
                m = cand[0];
#pragma unroll
                for (int t = 1; t < 32; ++t) m = max(m, cand[t]);
            } else {
                // a picked token (0) must lose the min scan: compare key - 1, which wraps 0 to the top
                m = cand[0] - 1u;
#pragma unroll
                for (int t = 1; t < 32; ++t) m = min(m, cand[t] - 1u);
                m += 1u;
            }
            bool found = false;
            int tok = 0;
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                const bool hit = !found && cand[t] == m;
                if (hit) { tok = t; cand[t] = 0u; }
                found |= hit;
            }
            pick_key[r] = m;
            pick_tok[r] = tok;
            omask |= 1u << tok;
        }
        // ---- base affine over the tokens that were not picked ----
        kmax = cand[0]; kmin = cand[0] - 1u;
#pragma unroll
        for (int t = 1; t < 32; ++t) { kmax = max(kmax, cand[t]); kmin = min(kmin, cand[t] - 1u); }
        kmin += 1u;
    }
    const float mn = key_f32(kmin), mx = key_f32(kmax);
    int e;
    const float scale = snap_scale(__fsub_rn(mx, mn), p.use_pow2, p.scale_kind, e);
    const float zp = store_f32 ? mn : bf16_round_f32(mn);
    // dividing by a power of two and multiplying by its reciprocal round identically
    const bool by_mul = p.use_pow2 && e >= -126 && e <= 126;
    const float inv = __uint_as_float((uint32_t)(by_mul ? 127 - e : 127) << 23);
    uint32_t cw0 = 0, cw1 = 0;                // this channel's codes, token t at bits 2t
    if (__all_sync(0xFFFFFFFFu, by_mul)) {    // the usual case, without a division in sight
        // clamp, then add 1.5 * 2^23: the code sits in the low bits of the sum's pattern 0x4B400000 + code.  The
        // patterns are accumulated shifted as they are; what the constant part adds up to (mod 2^32) leaves once.
        constexpr uint32_t MAGIC = 0x4B400000u;
        uint32_t magic_sum = 0;
#pragma unroll
        for (int t = 0; t < 16; ++t) magic_sum += MAGIC << (2 * t);
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            const float c = fminf(fmaxf(__fmul_rn(__fsub_rn(x[t], zp), inv), 0.f), 3.f);       // NaN -> 0
            const uint32_t bits = __float_as_uint(__fadd_rn(c, 12582912.f));
            if (t < 16) cw0 = bits * (1u << (2 * t)) + cw0;
            else cw1 = bits * (1u << (2 * (t - 16))) + cw1;
        }
        cw0 -= magic_sum;
        cw1 -= magic_sum;
    } else {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            const float d = __fsub_rn(x[t], zp);
            const uint32_t c = code_0_3(by_mul ? __fmul_rn(d, inv) : __fdiv_rn(d, scale));
            if (t < 16) cw0 = c * (1u << (2 * t)) + cw0;
            else cw1 = c * (1u << (2 * (t - 16))) + cw1;
        }
    }
    // ---- outlier values ----
    float ms = 0.f, mc = 0.f;
    uint32_t val = 0;
    if (K > 0) {
        if (p.outlier_map) {
            uint32_t okmin = pick_key[0], okmax = pick_key[0];
#pragma unroll
            for (int r = 1; r < K; ++r) { okmin = min(okmin, pick_key[r]); okmax = max(okmax, pick_key[r]); }
            const float omn = key_f32(okmin), omx = key_f32(okmax);
            mc = __fmul_rn(__fadd_rn(omx, omn), 0.5f);
            // the reference evaluates 12.0 / range as reciprocal(range) * 12
            ms = __fmul_rn(__frcp_rn(fmaxf(__fsub_rn(omx, omn), 1e-8f)), 12.0f);
            if (!store_f32) { mc = bf16_round_f32(mc); ms = bf16_round_f32(ms); }
        }
#pragma unroll
        for (int r = 0; r < K; ++r) {
            const float xo = key_f32(pick_key[r]);            // the picked value (-0.0 reads back as +0.0: same code)
            const float mapped = p.outlier_map ? __fmul_rn(__fsub_rn(xo, mc), ms) : __fdiv_rn(__fsub_rn(xo, zp), scale);
            const uint32_t fp4 = (uint32_t)fp4_encode_tbl(mapped, c_fp4_thresh);
            const int rank = __popc(omask & ((1u << pick_tok[r]) - 1u));
            val |= fp4 << (4 * rank);
        }
    }
    // ---- per-channel planes ----
    // With head_dim 128 the four warps of the block hold the four channel blocks of one (group, head): their plane
    // entries go through shared memory and leave as whole 16-byte pieces of contiguous rows (the standard planes:
    // int8 exponents, bf16 zero-points and map), one plane per warp.  Other shapes write lane by lane.
    __shared__ __align__(16) uint8_t s_rows[PACK_WARPS == 4 ? 128 * (1 + 2 + 2 + 2 + 4 + 4) : 16];
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(p.k_scale) | reinterpret_cast<uintptr_t>(p.k_zp) | reinterpret_cast<uintptr_t>(p.k_mapscale) |
                             reinterpret_cast<uintptr_t>(p.k_mapcenter) | reinterpret_cast<uintptr_t>(p.k_obmp) | reinterpret_cast<uintptr_t>(p.k_oval)) & 15u) == 0;
    const bool staged = nblk == PACK_WARPS && p.scale_kind == OMMX_SCALE_INT8_EXP && K > 0 && p.outlier_map && NB <= 4 && aligned16;
    if (staged) {
        // every warp of the block is here: g, h and the pool decisions above are the same for all four
        const int d = blk * 32 + lane;
        s_rows[d] = (uint8_t)(int8_t)e;
        reinterpret_cast<uint16_t *>(s_rows + 128)[d] = (uint16_t)f32_to_bf16_bits(zp);
        reinterpret_cast<uint16_t *>(s_rows + 384)[d] = (uint16_t)f32_to_bf16_bits(ms);
        reinterpret_cast<uint16_t *>(s_rows + 640)[d] = (uint16_t)f32_to_bf16_bits(mc);
        reinterpret_cast<uint32_t *>(s_rows + 896)[d] = omask;
#pragma unroll
        for (int i = 0; i < NB; ++i) s_rows[1408 + d * NB + i] = (uint8_t)(val >> (8 * i));
        __syncthreads();
        if (slot_ok) {
            const int64_t row = ((int64_t)slot * p.H + h) * D;           // first channel of the (slot, head) row
            const uint4 *src = reinterpret_cast<const uint4 *>(s_rows);
            if (warp == 0) {
                if (lane < 8) reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.k_scale) + row)[lane] = src[lane];
                else if (lane < 24) reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.k_zp) + 2 * row)[lane - 8] = src[lane];
            } else if (warp == 1) {
                if (lane < 16) reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.k_mapscale) + 2 * row)[lane] = src[24 + lane];
                else reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.k_mapcenter) + 2 * row)[lane - 16] = src[40 + lane - 16];
            } else if (warp == 2) {
                reinterpret_cast<uint4 *>(p.k_obmp + 4 * row)[lane] = src[56 + lane];
            } else {
                // 128 * NB bytes: a multiple of 16 only for even NB; the row start is 16-byte aligned when 128 * NB is
                for (int i = lane; i < 8 * NB; i += 32) reinterpret_cast<uint4 *>(p.k_oval + row * NB)[i] = src[88 + i];
            }
        }
    } else if (slot_ok) {
        const int64_t off = ((int64_t)slot * p.H + h) * D + blk * 32 + lane;
        if (p.scale_kind == OMMX_SCALE_INT8_EXP) reinterpret_cast<int8_t *>(p.k_scale)[off] = (int8_t)e;
        else if (p.scale_kind == OMMX_SCALE_BF16) reinterpret_cast<uint16_t *>(p.k_scale)[off] = (uint16_t)f32_to_bf16_bits(scale);
        else reinterpret_cast<float *>(p.k_scale)[off] = scale;
        if (store_f32) reinterpret_cast<float *>(p.k_zp)[off] = zp;
        else reinterpret_cast<uint16_t *>(p.k_zp)[off] = (uint16_t)f32_to_bf16_bits(zp);
        if (K > 0) {
            if (p.outlier_map) {
                if (store_f32) {
                    reinterpret_cast<float *>(p.k_mapscale)[off] = ms;
                    reinterpret_cast<float *>(p.k_mapcenter)[off] = mc;
                } else {
                    reinterpret_cast<uint16_t *>(p.k_mapscale)[off] = (uint16_t)f32_to_bf16_bits(ms);
                    reinterpret_cast<uint16_t *>(p.k_mapcenter)[off] = (uint16_t)f32_to_bf16_bits(mc);
                }
            }
            reinterpret_cast<uint32_t *>(p.k_obmp)[off] = omask;
#pragma unroll
            for (int i = 0; i < NB; ++i) p.k_oval[off * NB + i] = (uint8_t)(val >> (8 * i));
        }
    }
    if (bad) or_status(p.status, OMMX_ST_NONFINITE);

    // ---- codes: lane-major (channel, 32 tokens) -> token-major (token, 32 channels) ----
    // Stage s swaps element (lane, c) having lane bit s clear and c bit s set with element (lane^s, c^s).
    {
        const uint32_t send = (lane & 16) ? cw0 : cw1;
        const uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, send, 16);
        if (lane & 16) cw0 = got; else cw1 = got;
    }
    {
        const uint32_t g0 = __shfl_xor_sync(0xFFFFFFFFu, cw0, 8), g1 = __shfl_xor_sync(0xFFFFFFFFu, cw1, 8);
        const uint32_t sel = (lane & 8) ? 0x3276u : 0x5410u;
        cw0 = __byte_perm(cw0, g0, sel); cw1 = __byte_perm(cw1, g1, sel);
    }
    {
        const uint32_t g0 = __shfl_xor_sync(0xFFFFFFFFu, cw0, 4), g1 = __shfl_xor_sync(0xFFFFFFFFu, cw1, 4);
        const uint32_t sel = (lane & 4) ? 0x3715u : 0x6240u;
        cw0 = __byte_perm(cw0, g0, sel); cw1 = __byte_perm(cw1, g1, sel);
    }
    {
        const uint32_t g0 = __shfl_xor_sync(0xFFFFFFFFu, cw0, 2), g1 = __shfl_xor_sync(0xFFFFFFFFu, cw1, 2);
        if (lane & 2) { cw0 = (cw0 & 0xF0F0F0F0u) | ((g0 >> 4) & 0x0F0F0F0Fu); cw1 = (cw1 & 0xF0F0F0F0u) | ((g1 >> 4) & 0x0F0F0F0Fu); }
        else          { cw0 = (cw0 & 0x0F0F0F0Fu) | ((g0 << 4) & 0xF0F0F0F0u); cw1 = (cw1 & 0x0F0F0F0Fu) | ((g1 << 4) & 0xF0F0F0F0u); }
    }
    {
        const uint32_t g0 = __shfl_xor_sync(0xFFFFFFFFu, cw0, 1), g1 = __shfl_xor_sync(0xFFFFFFFFu, cw1, 1);
        if (lane & 1) { cw0 = (cw0 & 0xCCCCCCCCu) | ((g0 >> 2) & 0x33333333u); cw1 = (cw1 & 0xCCCCCCCCu) | ((g1 >> 2) & 0x33333333u); }
        else          { cw0 = (cw0 & 0x33333333u) | ((g0 << 2) & 0xCCCCCCCCu); cw1 = (cw1 & 0x33333333u) | ((g1 << 2) & 0xCCCCCCCCu); }
    }
    // lane = token now: its 8 code bytes of this channel block
    const int ps = p.page_size;
    const int tok = grp * 32 + lane;
    int page = tok / ps;
    if (p.pool.seq) page = p.pool.r2t[seq_slot * p.pool.pages_per_seq + page];
    else if (p.dst_pages) page = p.dst_pages[page];
    const bool page_ok = (page >= 0 && page < p.num_pages);
    if (!page_ok) or_status(p.status, OMMX_ST_BAD_PAGE);
    if (page_ok) {
        uint8_t *dst = p.k_base + (((int64_t)page * ps + (tok % ps)) * p.H + h) * (D / 4) + 8 * blk;
        *reinterpret_cast<uint2 *>(dst) = make_uint2(cw0, cw1);
    }
}

struct PackVParams {
    PoolSrc pool;
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
    int t = (int)(idx / ((int64_t)ngv * p.H));
    const T *row = reinterpret_cast<const T *>(p.v) + (int64_t)h * p.stride_head + cg * 32;
    int seq_slot = 0;
    if (p.pool.seq) {
        const int i = t / 32, tt = t % 32;                              // batch row, token inside the completed group
        seq_slot = pool_slot(p.pool, i);
        if (seq_slot < 0 || seq_slot >= p.pool.num_seqs) return;
        const int pos = pool_pos(p.pool, i, seq_slot);
        const int grp = pool_groups_at(p.pool, pos);
        if (pool_groups_at(p.pool, pos + 1) == grp) return;
        if (pool_row_refused(p.pool, seq_slot, pos + 1)) { or_status(p.status, OMMX_ST_BAD_LENGTH); return; }
        const int rec = p.pool.ring_cap - p.pool.sink;
        const int rr = (grp * 32 + tt) % rec;
        row += (int64_t)(seq_slot * p.pool.ring_cap + p.pool.sink + rr) * p.stride_token;
        t = grp * 32 + tt;                                              // token index inside the sequence's packed part
    } else {
        row += (int64_t)t * p.stride_token;
    }
    float x[32];
    bool bad = false;
    if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
        // 64 contiguous bytes: four 16-byte loads
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint4 w = reinterpret_cast<const uint4 *>(row)[v];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x[8 * v + 2 * i] = bits16_as_f32<T>(ww[i] & 0xFFFFu);
                x[8 * v + 2 * i + 1] = bits16_as_f32<T>(ww[i] >> 16);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = load_as_f32(row + i);
    }
#pragma unroll
    for (int i = 0; i < 32; ++i)
        if (!isfinite(x[i])) bad = true;
    float mn = x[0], mx = x[0];
#pragma unroll
    for (int i = 1; i < 32; ++i) { mn = fminf(mn, x[i]); mx = fmaxf(mx, x[i]); }
    mn += 0.0f;
    int e;
    const float scale = snap_scale(__fsub_rn(mx, mn), p.use_pow2, p.scale_kind, e);
    const bool store_f32 = (p.scale_kind == OMMX_SCALE_F32);
    const float zp = store_f32 ? mn : bf16_round_f32(mn);
    // dividing by a power of two and multiplying by its reciprocal round identically
    const bool by_mul = p.use_pow2 && e >= -126 && e <= 126;
    const float inv = __uint_as_float((uint32_t)(by_mul ? 127 - e : 127) << 23);
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float d = __fsub_rn(x[i], zp);
        const uint32_t c = code_0_3(by_mul ? __fmul_rn(d, inv) : __fdiv_rn(d, scale));
        if (i < 16) w0 = c * (1u << (2 * i)) + w0; else w1 = c * (1u << (2 * (i - 16))) + w1;
    }
    if (bad) or_status(p.status, OMMX_ST_NONFINITE);
    int page = t / p.page_size;
    if (p.pool.seq) page = p.pool.r2t[seq_slot * p.pool.pages_per_seq + page];
    else if (p.dst_pages) page = p.dst_pages[page];
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
    memset(&kp.pool, 0, sizeof(kp.pool));
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
    // the lane-per-channel kernel serves the signed rule with the usual outlier counts; everything else
    // (absolute selection, odd or large k) goes through the warp-reduction kernel
    const int lane_units = kp.num_groups * kp.H * (kp.D / 32);
    const unsigned lane_grid = (unsigned)((lane_units + PACK_WARPS - 1) / PACK_WARPS);
    const bool k_base_8 = (((uintptr_t)pl.k_base & 7) == 0);
    const int ksel = (kp.select_signed && k_base_8) ? kp.k_out : -1;
    if (units > 0) {
        switch (ksel) {
            case 0: pack_k_lane_kernel<T, 0, 0><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            case 2: pack_k_lane_kernel<T, 1, 1><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            case 4: pack_k_lane_kernel<T, 2, 2><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            case 6: pack_k_lane_kernel<T, 3, 3><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            case 8: pack_k_lane_kernel<T, 4, 4><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            default: pack_k_kernel<T><<<(units + PACK_WARPS - 1) / PACK_WARPS, PACK_WARPS * 32, 0, st>>>(kp); break;
        }
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    PackVParams vp;
    memset(&vp.pool, 0, sizeof(vp.pool));
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

// ---------------------------------------------------------------------------------------------
// Device-resident decode-step store (reference: MultiSeqKVPool.append_decode_device /
// decode_inputs_device, attention/kv_pool.py:440-488, :1048-1105; ring copies
// attention/kv_store_ops.py:22-57).  Four fixed-shape launches, no host synchronisation:
//   kv_ring_write_kernel   new row -> ring row of position seq
//   pack_k_lane_kernel     } pool source: every batch row whose step completed a 32-token group
//   pack_v_kernel          } packs it from the ring into its next pages / group slot; the rest return
//   kv_finalize_kernel     seq += 1, packed / residual lengths, residual rows gathered for the decode call
// ---------------------------------------------------------------------------------------------
struct StoreParams {
    PoolSrc pool;
    __nv_bfloat16 *k_hist, *v_hist;
    const __nv_bfloat16 *k_new, *v_new;
    int64_t new_sb, new_sh;
    int32_t H, D, num_seqs, advance;
    __nv_bfloat16 *k_tail, *v_tail;
    int32_t max_tail;
    int32_t *b_seq_len, *b_tail_len, *seq_len, *status;
};

__device__ __forceinline__ int ring_row(const PoolSrc &ps, int pos) {
    return pos < ps.sink ? pos : ps.sink + (pos - ps.sink) % (ps.ring_cap - ps.sink);
}

// grid (batch), 128 threads: one new K row and one new V row of H*D bf16 each
__global__ void __launch_bounds__(128) kv_ring_write_kernel(StoreParams p) {
    const int i = blockIdx.x;
    const int r = pool_slot(p.pool, i);
    if (r < 0 || r >= p.num_seqs) { if (threadIdx.x == 0) or_status(p.status, OMMX_ST_BAD_GROUP); return; }
    const int pos = pool_pos(p.pool, i, r);
    if (pos < 0 || pool_row_refused(p.pool, r, pos + 1)) { if (threadIdx.x == 0) or_status(p.status, OMMX_ST_BAD_LENGTH); return; }
    const int64_t dst = ((int64_t)r * p.pool.ring_cap + ring_row(p.pool, pos)) * p.H * p.D;
    for (int x = threadIdx.x; x < p.H * p.D; x += blockDim.x) {
        const int h = x / p.D, c = x - h * p.D;
        p.k_hist[dst + x] = p.k_new[(int64_t)i * p.new_sb + (int64_t)h * p.new_sh + c];
        p.v_hist[dst + x] = p.v_new[(int64_t)i * p.new_sb + (int64_t)h * p.new_sh + c];
    }
}

// grid (batch, rows): block (i, y) copies residual rows y, y + gridDim.y, ...; block (i, 0) also advances
// the sequence and writes the two lengths.  Every block derives the lengths from the same old value.
__global__ void __launch_bounds__(128) kv_finalize_kernel(StoreParams p) {
    const int i = blockIdx.x;
    const int r = pool_slot(p.pool, i);
    if (r < 0 || r >= p.num_seqs) return;
    const int old = pool_pos(p.pool, i, r);
    const int seq = old + ((p.advance && old >= 0 && !pool_row_refused(p.pool, r, old + 1)) ? 1 : 0);
    const int sink = p.pool.sink;
    const int spare = seq - sink - p.pool.recent;
    const int boundary = spare > 0 ? sink + spare / 32 * 32 : min(sink, seq);
    const int n_sink = min(sink, seq), n_rec = max(seq - boundary, 0);
    // a residual buffer too small for sink + recent + a partial group would silently drop the newest rows
    if (n_sink + n_rec > p.max_tail && (p.k_tail || p.b_tail_len) && blockIdx.y == 0 && threadIdx.x == 0)
        or_status(p.status, OMMX_ST_BAD_LENGTH);
    const int n_tail = min(n_sink + n_rec, p.max_tail);
    if (p.k_tail && p.v_tail) {
        const int HD = p.H * p.D;
        for (int row = blockIdx.y; row < n_tail; row += gridDim.y) {
            const int pos = row < n_sink ? row : boundary + (row - n_sink);
            const uint4 *ks = reinterpret_cast<const uint4 *>(p.k_hist + ((int64_t)r * p.pool.ring_cap + ring_row(p.pool, pos)) * HD);
            const uint4 *vs = reinterpret_cast<const uint4 *>(p.v_hist + ((int64_t)r * p.pool.ring_cap + ring_row(p.pool, pos)) * HD);
            uint4 *kd = reinterpret_cast<uint4 *>(p.k_tail + ((int64_t)i * p.max_tail + row) * HD);
            uint4 *vd = reinterpret_cast<uint4 *>(p.v_tail + ((int64_t)i * p.max_tail + row) * HD);
            for (int x = threadIdx.x; x < HD / 8; x += blockDim.x) { kd[x] = ks[x]; vd[x] = vs[x]; }
        }
    }
    if (blockIdx.y == 0 && threadIdx.x == 0) {
        if (p.b_seq_len) p.b_seq_len[i] = max(boundary - sink, 0);
        if (p.b_tail_len) p.b_tail_len[i] = n_tail;
    }
}

// seq_len is advanced by its own one-thread-per-row kernel after every reader of the old value has run
__global__ void kv_advance_kernel(StoreParams p, int batch) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch) return;
    const int r = pool_slot(p.pool, i);
    if (r >= 0 && r < p.num_seqs) {
        const int old = pool_pos(p.pool, i, r);
        if (old >= 0 && !pool_row_refused(p.pool, r, old + 1)) p.seq_len[r] = old + 1;
    }
}

// Residual rows by caller-supplied absolute token positions (the reference's _kv_gather_tail,
// attention/kv_store_ops.py:42-57): grid (batch, rows); row y of batch row i is token idx[i*T + y] of
// sequence slot sel[i], read from its ring row.  A negative position or a slot outside the pool is
// reported and the row is zero-filled (the reference asserts on the device).
struct GatherParams {
    const __nv_bfloat16 *k_hist, *v_hist;
    const void *sel, *idx;
    int32_t idx64, T, HD, ring_cap, sink, num_seqs;
    __nv_bfloat16 *k_tail, *v_tail;
    int32_t *status;
};
__global__ void __launch_bounds__(128) kv_gather_tail_kernel(GatherParams p) {
    const int i = blockIdx.x;
    const int r = p.sel ? pool_index(p.sel, p.idx64, i) : i;
    const bool slot_ok = r >= 0 && r < p.num_seqs;
    for (int row = blockIdx.y; row < p.T; row += gridDim.y) {
        const int pos = pool_index(p.idx, p.idx64, i * p.T + row);
        const bool ok = slot_ok && pos >= 0;
        if (!ok && threadIdx.x == 0) or_status(p.status, slot_ok ? OMMX_ST_BAD_LENGTH : OMMX_ST_BAD_GROUP);
        const int rr = pos < p.sink ? pos : p.sink + (pos - p.sink) % (p.ring_cap - p.sink);
        const uint4 *ks = reinterpret_cast<const uint4 *>(p.k_hist + ((int64_t)(ok ? r : 0) * p.ring_cap + (ok ? rr : 0)) * p.HD);
        const uint4 *vs = reinterpret_cast<const uint4 *>(p.v_hist + ((int64_t)(ok ? r : 0) * p.ring_cap + (ok ? rr : 0)) * p.HD);
        uint4 *kd = reinterpret_cast<uint4 *>(p.k_tail + ((int64_t)i * p.T + row) * p.HD);
        uint4 *vd = reinterpret_cast<uint4 *>(p.v_tail + ((int64_t)i * p.T + row) * p.HD);
        for (int x = threadIdx.x; x < p.HD / 8; x += blockDim.x) {
            kd[x] = ok ? ks[x] : make_uint4(0, 0, 0, 0);
            vd[x] = ok ? vs[x] : make_uint4(0, 0, 0, 0);
        }
    }
}

static int launch_append(const ommx_kv_append_args *a, cudaStream_t st) {
    const ommx_kv_pool &pool = a->pool;
    const ommx_kv_planes &pl = pool.planes;
    StoreParams sp;
    sp.pool.seq = pool.seq_len; sp.pool.slots = a->slots; sp.pool.r2t = pool.req_to_token; sp.pool.r2g = pool.req_to_group;
    sp.pool.ring_cap = pool.ring_cap; sp.pool.sink = pool.sink_tokens; sp.pool.recent = pool.recent_window;
    sp.pool.groups_per_seq = pool.groups_per_seq; sp.pool.pages_per_seq = pool.pages_per_seq;
    sp.pool.num_seqs = pool.num_seqs; sp.pool.pages_per_group = 32 / pl.page_size;
    sp.pool.wpos = a->write_pos; sp.pool.idx64 = a->index_is_int64 ? 1 : 0;
    sp.k_hist = (__nv_bfloat16 *)pool.k_hist; sp.v_hist = (__nv_bfloat16 *)pool.v_hist;
    sp.k_new = (const __nv_bfloat16 *)a->k_new; sp.v_new = (const __nv_bfloat16 *)a->v_new;
    sp.new_sb = a->new_stride_b; sp.new_sh = a->new_stride_h;
    sp.H = pl.n_kv_heads; sp.D = pl.head_dim; sp.num_seqs = pool.num_seqs; sp.advance = a->advance ? 1 : 0;
    sp.k_tail = (__nv_bfloat16 *)a->k_tail; sp.v_tail = (__nv_bfloat16 *)a->v_tail; sp.max_tail = a->max_tail;
    sp.b_seq_len = a->b_seq_len; sp.b_tail_len = a->b_tail_len; sp.seq_len = pool.seq_len; sp.status = a->status;
    const int B = a->batch;
    if (a->advance) {
        kv_ring_write_kernel<<<B, 128, 0, st>>>(sp);
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
        PackKParams kp;
        kp.pool = sp.pool;
        kp.k = pool.k_hist; kp.stride_token = (int64_t)sp.H * sp.D; kp.stride_head = sp.D;
        kp.num_groups = B; kp.H = sp.H; kp.D = sp.D; kp.page_size = pl.page_size;
        kp.dst_pages = nullptr; kp.dst_groups = nullptr;
        kp.num_pages = pl.num_pages; kp.num_group_slots = pl.num_group_slots;
        kp.k_out = pl.outliers_per_vector; kp.select_signed = 1; kp.use_pow2 = a->use_pow2;
        kp.outlier_map = pl.kv_outlier_map; kp.scale_kind = pl.scale_kind;
        kp.k_base = (uint8_t *)pl.k_base; kp.k_scale = pl.k_scale; kp.k_zp = pl.k_zp;
        kp.k_mapscale = pl.k_mapscale; kp.k_mapcenter = pl.k_mapcenter;
        kp.k_obmp = (uint8_t *)pl.k_obmp; kp.k_oval = (uint8_t *)pl.k_oval; kp.status = a->status;
        const int lane_units = B * kp.H * (kp.D / 32);
        const unsigned lane_grid = (unsigned)((lane_units + PACK_WARPS - 1) / PACK_WARPS);
        typedef __nv_bfloat16 T;
        switch (kp.k_out) {
            case 0: pack_k_lane_kernel<T, 0, 0><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            case 2: pack_k_lane_kernel<T, 1, 1><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            case 4: pack_k_lane_kernel<T, 2, 2><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            case 6: pack_k_lane_kernel<T, 3, 3><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
            default: pack_k_lane_kernel<T, 4, 4><<<lane_grid, PACK_WARPS * 32, 0, st>>>(kp); break;
        }
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
        PackVParams vp;
        vp.pool = sp.pool;
        vp.v = pool.v_hist; vp.stride_token = kp.stride_token; vp.stride_head = sp.D;
        vp.num_tokens = B * 32; vp.H = sp.H; vp.D = sp.D; vp.page_size = pl.page_size;
        vp.dst_pages = nullptr; vp.num_pages = pl.num_pages; vp.use_pow2 = a->use_pow2; vp.scale_kind = pl.scale_kind;
        vp.v_main = (uint8_t *)pl.v_main; vp.v_scale = pl.v_scale; vp.v_zp = pl.v_zp; vp.status = a->status;
        const int64_t nthreads = (int64_t)vp.num_tokens * vp.H * (vp.D / 32);
        pack_v_kernel<T><<<(unsigned)((nthreads + 127) / 128), 128, 0, st>>>(vp);
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    if (a->b_seq_len || a->b_tail_len || (a->k_tail && a->v_tail)) {
        dim3 grid(B, (a->k_tail && a->v_tail) ? 8 : 1);
        kv_finalize_kernel<<<grid, 128, 0, st>>>(sp);
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    if (a->advance == 1) {
        kv_advance_kernel<<<(B + 127) / 128, 128, 0, st>>>(sp, B);
        OMMX_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    return 0;
}

}  // namespace ommx

namespace ommx {
// One thread per frame.  relidx7 (ommx_gpu_serve/attention/codec.py:91-130 of the reference): the k token positions of
// a frame, ascending, 7 bits each, LSB first, in ceil(7k/8) bytes.
__global__ void outlier_index_convert_kernel(const uint8_t *src, uint8_t *dst, int64_t frames, int k, int to_relidx7, int32_t *status) {
    const int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= frames) return;
    const int nbi = (7 * k + 7) / 8;
    if (to_relidx7) {
        uint32_t bits = (uint32_t)src[4 * f] | ((uint32_t)src[4 * f + 1] << 8) | ((uint32_t)src[4 * f + 2] << 16) | ((uint32_t)src[4 * f + 3] << 24);
        if (__popc(bits) != k) or_status(status, OMMX_ST_BAD_GROUP);
        unsigned long long lo = 0, hi = 0;                       // 7k <= 112 bits
        int r = 0;
        while (bits && r < k) {
            const int pz = __ffs(bits) - 1;
            bits &= bits - 1;
            const int bp = 7 * r;
            if (bp < 64) { lo |= (unsigned long long)pz << bp; if (bp > 57) hi |= (unsigned long long)pz >> (64 - bp); }
            else hi |= (unsigned long long)pz << (bp - 64);
            ++r;
        }
        for (int i = 0; i < nbi; ++i) dst[f * nbi + i] = (uint8_t)((i < 8 ? lo >> (8 * i) : hi >> (8 * (i - 8))) & 0xFFu);
    } else {
        unsigned long long lo = 0, hi = 0;
        for (int i = 0; i < nbi; ++i) {
            const unsigned long long b = src[f * nbi + i];
            if (i < 8) lo |= b << (8 * i); else hi |= b << (8 * (i - 8));
        }
        uint32_t bits = 0;
        for (int r = 0; r < k; ++r) {
            const int bp = 7 * r;
            unsigned long long v = bp < 64 ? lo >> bp : hi >> (bp - 64);
            if (bp < 64 && bp > 57) v |= hi << (64 - bp);
            const uint32_t pz = (uint32_t)(v & 0x7Fu);
            if (pz > 31u || (bits >> pz) & 1u) or_status(status, OMMX_ST_BAD_GROUP);
            else bits |= 1u << pz;
        }
        dst[4 * f] = (uint8_t)bits; dst[4 * f + 1] = (uint8_t)(bits >> 8); dst[4 * f + 2] = (uint8_t)(bits >> 16); dst[4 * f + 3] = (uint8_t)(bits >> 24);
    }
}
}  // namespace ommx

extern "C" int ommx_b200_outlier_index_convert(const void *src, void *dst, int64_t frames, int32_t k, int32_t to_relidx7,
                                               int32_t *status, void *stream) {
    using namespace ommx;
    if (!src || !dst) return fail(OMMX_E_ARG, "outlier_index_convert: null plane");
    if (frames < 0 || k < 1 || k > 16) return fail(OMMX_E_ARG, "outlier_index_convert: frames=%lld k=%d (k must be 1..16)", (long long)frames, k);
    if (frames == 0) return 0;
    outlier_index_convert_kernel<<<(unsigned)((frames + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t *)src, (uint8_t *)dst, frames, k, to_relidx7 ? 1 : 0, status);
    OMMX_CUDA_TRY(cudaGetLastError());
    count_launch();
    return 0;
}

extern "C" int ommx_b200_pack_kv(const ommx_pack_args *a, void *stream) {
    using namespace ommx;
    if (!a) return fail(OMMX_E_ARG, "pack: null args");
    const ommx_kv_planes &pl = a->planes;
    if (pl.outlier_index != OMMX_OIDX_BITMASK)
        return fail(OMMX_E_UNSUPPORTED, "pack: the store kernels write the flat bitmask (re-encode with ommx_b200_outlier_index_convert)");
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

extern "C" int ommx_b200_kv_append_decode(const ommx_kv_append_args *a, void *stream) {
    using namespace ommx;
    if (!a) return fail(OMMX_E_ARG, "kv_append: null args");
    const ommx_kv_pool &pool = a->pool;
    const ommx_kv_planes &pl = pool.planes;
    if (pl.outlier_index != OMMX_OIDX_BITMASK) return fail(OMMX_E_UNSUPPORTED, "kv_append: the store kernels write the flat bitmask");
    if (a->batch <= 0) return fail(OMMX_E_ARG, "kv_append: batch=%d", a->batch);
    if (!pool.k_hist || !pool.v_hist || !pool.seq_len || !pool.req_to_token || !pool.req_to_group)
        return fail(OMMX_E_ARG, "kv_append: ring, seq_len and the two tables must not be null");
    if (pool.num_seqs <= 0 || pool.sink_tokens < 0 || pool.recent_window < 0)
        return fail(OMMX_E_ARG, "kv_append: num_seqs=%d sink=%d recent=%d", pool.num_seqs, pool.sink_tokens, pool.recent_window);
    if (pool.ring_cap - pool.sink_tokens < pool.recent_window + 32)
        return fail(OMMX_E_ARG, "kv_append: ring_cap=%d must hold sink + recent + 32 rows (%d)", pool.ring_cap,
                    pool.sink_tokens + pool.recent_window + 32);
    if (pool.pages_per_seq <= 0 || pool.groups_per_seq <= 0)
        return fail(OMMX_E_ARG, "kv_append: pages_per_seq/groups_per_seq must be positive");
    if (pl.head_dim % 32 != 0 || pl.head_dim <= 0 || pl.n_kv_heads <= 0)
        return fail(OMMX_E_UNSUPPORTED, "kv_append: head_dim=%d n_kv_heads=%d", pl.head_dim, pl.n_kv_heads);
    if (pl.page_size <= 0 || 32 % pl.page_size != 0)
        return fail(OMMX_E_ARG, "kv_append: page_size=%d must divide 32", pl.page_size);
    if (a->advance) {
        if (!a->k_new || !a->v_new) return fail(OMMX_E_ARG, "kv_append: k_new/v_new are null");
        if (a->outlier_select != 1)
            return fail(OMMX_E_UNSUPPORTED, "kv_append: only the signed outlier rule is served");
        const int k = pl.outliers_per_vector;
        if (k != 0 && k != 2 && k != 4 && k != 6 && k != 8)
            return fail(OMMX_E_UNSUPPORTED, "kv_append: outliers_per_vector=%d (served: 0, 2, 4, 6, 8)", k);
        if (pl.scale_kind == OMMX_SCALE_INT8_EXP && !a->use_pow2)
            return fail(OMMX_E_ARG, "kv_append: int8 exponent scales need use_pow2");
        if (!pl.k_base || !pl.k_scale || !pl.k_zp || !pl.v_main || !pl.v_scale || !pl.v_zp)
            return fail(OMMX_E_ARG, "kv_append: a destination plane is null");
        if (k > 0 && (!pl.k_obmp || !pl.k_oval)) return fail(OMMX_E_ARG, "kv_append: k>0 needs k_obmp and k_oval");
        if (k > 0 && pl.kv_outlier_map && (!pl.k_mapscale || !pl.k_mapcenter))
            return fail(OMMX_E_ARG, "kv_append: kv_outlier_map needs k_mapscale and k_mapcenter");
        if (((uintptr_t)pl.k_base & 7) || ((uintptr_t)pl.v_main & 7) || ((uintptr_t)pl.k_obmp & 3))
            return fail(OMMX_E_ARG, "kv_append: k_base/v_main must be 8-byte and k_obmp 4-byte aligned");
    }
    if ((a->k_tail != nullptr) != (a->v_tail != nullptr)) return fail(OMMX_E_ARG, "kv_append: k_tail and v_tail go together");
    if (a->k_tail && (a->max_tail <= 0 || (pl.n_kv_heads * pl.head_dim) % 8 != 0 ||
                      ((uintptr_t)a->k_tail & 15) || ((uintptr_t)a->v_tail & 15) ||
                      ((uintptr_t)pool.k_hist & 15) || ((uintptr_t)pool.v_hist & 15)))
        return fail(OMMX_E_ARG, "kv_append: residual buffers need max_tail > 0 and 16-byte alignment");
    return launch_append(a, (cudaStream_t)stream);
}

extern "C" int ommx_b200_kv_gather_tail(const ommx_kv_pool *pool, const void *sel, const void *tail_idx,
                                        int32_t index_is_int64, int32_t batch, int32_t rows,
                                        void *k_tail, void *v_tail, int32_t *status, void *stream) {
    using namespace ommx;
    if (!pool || !tail_idx || !k_tail || !v_tail) return fail(OMMX_E_ARG, "kv_gather_tail: null pointer");
    if (!pool->k_hist || !pool->v_hist) return fail(OMMX_E_ARG, "kv_gather_tail: the pool has no residual ring");
    if (batch <= 0 || rows <= 0) return fail(OMMX_E_ARG, "kv_gather_tail: batch=%d rows=%d", batch, rows);
    const int HD = pool->planes.n_kv_heads * pool->planes.head_dim;
    if (HD <= 0 || HD % 8 != 0 || ((uintptr_t)k_tail & 15) || ((uintptr_t)v_tail & 15) ||
        ((uintptr_t)pool->k_hist & 15) || ((uintptr_t)pool->v_hist & 15))
        return fail(OMMX_E_ARG, "kv_gather_tail: rows must be whole 16-byte pieces on 16-byte aligned buffers");
    if (pool->ring_cap - pool->sink_tokens <= 0) return fail(OMMX_E_ARG, "kv_gather_tail: ring_cap=%d sink=%d", pool->ring_cap, pool->sink_tokens);
    GatherParams g;
    g.k_hist = (const __nv_bfloat16 *)pool->k_hist; g.v_hist = (const __nv_bfloat16 *)pool->v_hist;
    g.sel = sel; g.idx = tail_idx; g.idx64 = index_is_int64 ? 1 : 0; g.T = rows; g.HD = HD;
    g.ring_cap = pool->ring_cap; g.sink = pool->sink_tokens; g.num_seqs = pool->num_seqs;
    g.k_tail = (__nv_bfloat16 *)k_tail; g.v_tail = (__nv_bfloat16 *)v_tail; g.status = status;
    kv_gather_tail_kernel<<<dim3(batch, rows < 8 ? rows : 8), 128, 0, (cudaStream_t)stream>>>(g);
    OMMX_CUDA_TRY(cudaGetLastError());
    count_launch();
    return 0;
}
