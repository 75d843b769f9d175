// Split-KV stage 1 on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
// Included by ommx_decode.cu after its PTX wrappers, S1Params and CopyDesc.
//
// Same contract as decode_stage1_kernel (it replaces _canonical_splitkv_stage1,
// ommx_gpu_serve/attention/paged_decode.py:1255-2284 of the reference): one CTA serves one
// (split, sequence) pair and all local kv heads of its token range.  What differs is where the
// arithmetic runs.  A (32-token group, kv head) UNIT is expanded by stateless decode warps into fp16
// operand tiles in shared memory; one thread issues tcgen05.mma on them; the logits and the output
// accumulate in tensor memory, so no warp carries accumulator registers or a dependent MMA chain:
//
//   producer warp    streams one group (all kv heads) per ring stage, as the register-operand kernel does.
//   decode warps     per (unit, channel quarter): K codes -> fp16 c * 2^-16 (a 2-bit field moved to bits 8..9
//                    of a half-word IS that subnormal: shift + mask, exact) into the K tile
//                    [4 units x 32 tokens][128 channels]; the unit's outliers written OVER their slots as
//                    code + bf16(value - base value) / scale, times 2^-16 - the reference's own rounding of the
//                    outlier delta, no delta tile (fp16 holds such an
//                    entry to 2^-8 of a code step; for channels with a large scale the rounding residual goes into
//                    one of 8 spare positions per channel half, whose B entries repeat the channel's); the query
//                    rows scaled by the unit's power-of-two K scales (B tile); the fp32 q.zp sums; V codes
//                    -> the V tile (channel-major, fields masked in place); V scale / zero-point factors.
//   MMA thread       logits  D[4x32 tokens][unit, head] = Ktile . Bq^T            (8 x tcgen05.mma, K = 16)
//                    output  O[128 channels][scale group, head] += Vtile . P'^T                  (2 per unit)
//                    where P' = P * 2^e_v of the column's scale group: a channel row reads the columns of its
//                    own scale group, the others are never looked at.
//   4 softmax warps  (one per unit of an item = one quarter of the tensor-memory lanes): logits from tensor
//                    memory, lane = token; per-head maximum by redux.sync; online softmax whose reference
//                    maximum moves only when the true one outgrows it by 2^4 (the accumulators are then
//                    rescaled in tensor memory by all four warps, each on its lane quarter); the P' tiles; the
//                    V zero-point term sum_t P * zp as per-lane fp32 partial sums, reduced once at the end.
//
// Numerics keep the reference's rounding points where they matter for its gate: bf16 q * sm_scale, exact
// code * 2^e products, fp32 q.zp from the raw query, fp32 accumulation, V as exact code * 2^e products with
// the outlier delta rounded to bf16, the zero-point bias of V summed apart.  Differences inside the gate: P is
// rounded to fp16, and an outlier of a channel whose scale is below 4 sits on the fp16 grid of the code tile
// (2^-8 of a code step).
#pragma once

namespace ommx {

constexpr int TC_WARPS = 24;
constexpr int TC_THREADS = TC_WARPS * 32;
constexpr int TC_W_PRODUCER = 0, TC_W_MMA = 1, TC_W_SOFTMAX = 4;     // softmax warps 4..7: lane quarter = warp & 3
constexpr int TC_NDW = TC_WARPS - 6;                                  // decode warps: 2, 3, 8..23
constexpr int TC_FBQ = 4;          // B tile entry = q_c * 2^(e_k + FBQ); logit = D * 2^(16 - FBQ)
constexpr int TC_FBV = 2;          // P' = P * 2^(e_v + FBV); output = D * 2^(24 - 2 slot - FBV)
constexpr float TC_RESCALE_LOG2 = 4.f;   // the reference maximum follows the true one once it is 2^4 behind
constexpr int TC_KCHUNKS = 18;     // 8-position chunks of a K tile row: 16 of channels + 2 of outlier residuals (one per channel half)
constexpr int TC_KTILE = TC_KCHUNKS * 2048, TC_VTILE = 32768, TC_UNIT_TILE = 8192;
constexpr int TC_FLAG_E = 2;       // channels whose K scale is 2^2 or more get their outliers' rounding residual carried too
constexpr int TC_RES_SHIFT = 10;   // residual entries are stored times 2^10, their B entries times 2^-10
constexpr int TC_MAX_STAGES = 8;
constexpr int TC_SIDE_VF = 0, TC_SIDE_VZ = 1024, TC_SIDE_QZ = 2048, TC_SIDE_BYTES = 2560;   // factors, zero-points, q.zp [unit][quarter][8]

// barrier slots (8 bytes each)
// A waiter tells phases apart by parity only, so it must never be two completions away from the one it asks for.
// The MMA thread and the softmax warps visit every item in order and need two barriers per event (item & 1).  The
// decode warps skip items (tasks are dealt round-robin), so the events they wait for - logits of item i-2 issued
// and consumed, probabilities of item i-2 written, output MMAs of item i-1 / i-2 landed - rotate over four.
constexpr int TB_FULL = 0, TB_EMPTY = TC_MAX_STAGES, TB_KREADY = 2 * TC_MAX_STAGES, TB_KFREE = TB_KREADY + 2,
              TB_VREADY = TB_KFREE + 4, TB_PVDONE = TB_VREADY + 2, TB_DQFULL = TB_PVDONE + 4, TB_DQFREE = TB_DQFULL + 2,
              TB_PREADY = TB_DQFREE + 2, TB_COUNT = TB_PREADY + 4;
// words after the barriers
constexpr int TM_TMEM = 0, TM_ABORT = 1, TM_NEED = 2 /* [2][4] */, TM_CORR = 10 /* [2][4][8] */, TM_FM = 74 /* [8][8] */,
              TM_FL = 138 /* [8][8] */, TM_FB = 202 /* [8][32] */, TM_WORDS = 458;

struct TcParams {
    S1Params s;
    int32_t nb;                      // output accumulator blocks in tensor memory: max(H, 4)
    int32_t nvb;                     // V tile buffers (1 or 2)
    int32_t tab_pages, tab_groups;   // capacity of the split's page / group-slot tables
    uint32_t o_ktile, o_vtile, o_bq, o_ptile, o_side, o_q16, o_qraw, o_lut, o_tab, o_bar, o_desc;
    uint32_t tmem_cols;
};

// ---- tcgen05 wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    // shared-memory matrix descriptor, no swizzle: start >> 4 | leading-dimension offset | stride offset | version 1
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | ((uint64_t)1 << 46);
}
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N, int a_mn_major, int b_mn_major) {
    // kind::f16 instruction descriptor: D = f32, A = B = f16, major-ness, N >> 3, M >> 4
    return (1u << 4) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t addr, uint32_t (&r)[N]) {
    static_assert(N == 4 || N == 8, "4 or 8 columns");
    if constexpr (N == 4)
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
    else
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tmem_st(uint32_t addr, const uint32_t (&r)[N]) {
    if constexpr (N == 4)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
    else
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float redux_max_f32(float x) {
    float y;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(y) : "f"(x));
    return y;
}
// probe without blocking / block for at most `ns` nanoseconds (the plain try_wait may block for an unspecified time)
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_ns(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint32_t dup16(uint32_t h) { return h | (h << 16); }
// fp16 bits of 2^(e + bias): 0 below the subnormal range of interest (e + bias < -14), clamped at 2^15
__device__ __forceinline__ uint32_t tc_pow2_f16(int e, int bias, bool &clamped, int limit = 30) {
    int u = e + 15 + bias;
    clamped = u > limit;
    u = min(u, limit);
    return u < 1 ? 0u : (uint32_t)u << 10;
}
constexpr int TC_VF_LIMIT = 15 + 11;   // P' = P * 2^(e_v + FBV) with P up to 2^4: the factor stays at or below 2^11
// channel held at position kpos of a K tile row (and row m of a V tile): a 32-bit code word yields its 16
// channels as the pairs (i, i + 8), i = 0..7, so positions 2i and 2i + 1 of each 16-block hold channels i and i + 8
__device__ __forceinline__ int tc_channel_of(int pos) { return (pos & ~15) + ((pos & 15) >> 1) + ((pos & 1) << 3); }
__device__ __forceinline__ int tc_pos_of(int ch) { return (ch & ~15) + ((ch & 7) << 1) + ((ch >> 3) & 1); }
__device__ __forceinline__ int tc_vslot(int m) { const int i = (m & 15) >> 1; return i < 5 ? i : i - 5; }

// Outliers of channel 32qt + lane of one unit, written over their slots of the K tile row by row (the codes of the
// quarter are in place).  KO > 0: the count is known, all gathers (bit walk, FP4 level, base code read back from the
// slot) are issued before the first store, so their latencies overlap; KO < 0: any count, one pass.
// Entry = (code + bf16(value - base value) / scale) * 2^-16: the reference adds to the base value code * scale + zp a
// delta rounded to bf16 (paged_decode.py:1923-1950), and the same rounding here keeps the two paths' noise in step.
// Channels with a scale of 2^TC_FLAG_E or more also carry the entry's rounding residual (times 2^10) in one of four
// spare positions of the quarter, whose B entries are the channel's own times 2^-10.
template <int KO>
__device__ __forceinline__ void tc_splice(const S1Params &p, const uint8_t *gb, uint8_t *ktile, uint8_t *bq, const uint16_t *s_q16,
                                          const float *s_lut, int h, int ub, int qt, int lane, int gqap, int n_qk, bool &clamped_any) {
    const int d = 32 * qt + lane;
    const int nb = p.nb;
    const int e_raw = (int)(int8_t)gb[p.o_ks + h * 128 + d];
    const float zp = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(gb + p.o_kz + h * 256 + 2 * d));
    uint32_t bits = *reinterpret_cast<const uint32_t *>(gb + p.o_bm + h * 512 + 4 * d);
    const uint8_t *sv = gb + p.o_ov + (h * 128 + d) * nb;
    const int e = min(max(e_raw, -126), 100);
    const float sc = __uint_as_float((uint32_t)(e + 127) << 23);
    const float inv_s = __uint_as_float((uint32_t)(127 - 16 - e) << 23);           // 2^-16 / scale
    float A = sc, Bc = zp;                                                          // shared map: value = level * scale + zp
    if (p.use_map) {                                                                // dedicated map: level / map scale + map centre
        A = __fdividef(1.f, bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(gb + p.o_ms + h * 256 + 2 * d)));
        Bc = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(gb + p.o_mc + h * 256 + 2 * d));
    }
    const uint32_t fm = __ballot_sync(0xFFFFFFFFu, e_raw >= TC_FLAG_E);
    const int slot = __popc(fm & ((1u << lane) - 1u));
    const bool res = e_raw >= TC_FLAG_E && slot < 4;
    const int kc = 16 + (qt >> 1), so = 8 * (qt & 1);                               // residual chunk, byte offset of this quarter's four slots
    *reinterpret_cast<uint2 *>(ktile + 16 * (32 * ub + lane) + kc * 2048 + so) = make_uint2(0u, 0u);
    uint8_t *bq_res = bq + 16 * (ub * gqap) + kc * (16 * n_qk) + so;
    if (lane < gqap) *reinterpret_cast<uint2 *>(bq_res + 16 * lane) = make_uint2(0u, 0u);
    __syncwarp();
    const int pos = tc_pos_of(d);
    uint8_t *col = ktile + 16 * (32 * ub) + (pos >> 3) * 2048 + (pos & 7) * 2;
    uint8_t *rcol = ktile + 16 * (32 * ub) + kc * 2048 + so + 2 * slot;
    if (res) {
        bool cl;
        const uint32_t f = tc_pow2_f16(e, TC_FBQ - TC_RES_SHIFT, cl);
        for (int j = 0; j < p.gqa; ++j)
            *reinterpret_cast<uint16_t *>(bq_res + 16 * j + 2 * slot) = (uint16_t)(hmul2_f16(s_q16[(h * gqap + j) * 128 + pos], f) & 0xFFFFu);
    }
    (void)clamped_any;
    auto entry = [&](float lvl, uint32_t cbits, int pz) {
        const float cf = (float)(cbits >> 8);
        const float delta = bf16_round_f32(fmaf(lvl, A, Bc) - fmaf(cf, sc, zp));
        const float X = fmaf(delta, inv_s, cf * 1.52587890625e-05f);                // (code + delta / scale) * 2^-16
        const uint32_t hbits = f16_bits_sat(X);
        *reinterpret_cast<uint16_t *>(col + 16 * pz) = (uint16_t)hbits;
        if (res) {
            const float back = __half2float(__ushort_as_half((unsigned short)hbits));
            *reinterpret_cast<uint16_t *>(rcol + 16 * pz) = (uint16_t)f16_bits_sat((X - back) * (float)(1 << TC_RES_SHIFT));
        }
    };
    if constexpr (KO > 0) {
        if (__popc(bits) != KO) { or_status(p.status, OMMX_ST_BAD_GROUP); return; }   // bitmask and value stream disagree
        uint32_t stream = 0;
#pragma unroll
        for (int i = 0; i < (KO + 1) / 2; ++i) stream |= (uint32_t)sv[i] << (8 * i);
        // batches of up to four: all gathers of a batch before its first store (more would cost registers)
#pragma unroll
        for (int top = KO - 1; top >= 0; top -= 4) {
            int pzs[4];
            float lvs[4];
            uint32_t cbs[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int r = top - q;
                if (r < 0) continue;
                const int pz = 31 - __clz(bits);
                bits ^= 1u << pz;
                pzs[q] = pz;
                lvs[q] = s_lut[(stream >> (4 * r)) & 0xFu];
                cbs[q] = *reinterpret_cast<const uint16_t *>(col + 16 * pz);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (top - q >= 0) entry(lvs[q], cbs[q], pzs[q]);
        }
    } else {
        int r = __popc(bits) - 1;
        if (r + 1 != p.k_out) or_status(p.status, OMMX_ST_BAD_GROUP);
        r = min(r, 2 * nb - 1);
        while (bits) {
            const int pz = 31 - __clz(bits);
            bits ^= 1u << pz;
            const uint32_t nib = ((uint32_t)sv[r >> 1] >> (4 * (r & 1))) & 0xFu;
            --r;
            entry(s_lut[nib], *reinterpret_cast<const uint16_t *>(col + 16 * pz), pz);
        }
    }
}

// =================================================================================================
template <int GQAP, bool NB8>
__global__ void __launch_bounds__(TC_THREADS, 1) decode_stage1_tc_kernel(const __grid_constant__ TcParams P) {
    const S1Params &p = P.s;
    constexpr int N_QK = 4 * GQAP;                   // logit columns: (unit in item, head)
    constexpr int N_PV = 4 * GQAP;                   // output columns: (V scale group, head)
    constexpr int BQ_BYTES = TC_KCHUNKS * 16 * N_QK;
    constexpr int PT_BYTES = N_PV * 64;              // one P' tile: N_PV rows x 32 tokens
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int split = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // placed while the previous kernel of the stream drains; no global memory is touched before this returns
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- split range (same rounding as the reference, paged_decode.py:1428-1432) ----
    const int seq = p.b_seq_len[b];
    if (seq <= 0) return;
    const int per = (((seq + p.S - 1) / p.S) + 31) / 32 * 32;
    const int t0 = split * per;
    const int t1 = min(t0 + per, seq);
    if (t1 <= t0) return;
    const int ntok = t1 - t0;
    const int ngroups = (ntok + 31) / 32;
    if (ngroups > P.tab_groups || ngroups * p.ppg > P.tab_pages) {
        if (threadIdx.x == 0) or_status(p.status, OMMX_ST_BAD_LENGTH);
        return;
    }
    const int H = p.H, NS = p.nstages, gqa = p.gqa;
    const int n_units = ngroups * H;
    const int n_items = (n_units + 3) >> 2;
    const int k_out = p.k_out;

    uint8_t *s_stage = smem;
    uint8_t *s_ktile = smem + P.o_ktile, *s_vtile = smem + P.o_vtile, *s_bq = smem + P.o_bq, *s_pt = smem + P.o_ptile;
    uint8_t *s_side = smem + P.o_side;
    uint16_t *s_q16 = reinterpret_cast<uint16_t *>(smem + P.o_q16), *s_qraw = reinterpret_cast<uint16_t *>(smem + P.o_qraw);
    float *s_lut = reinterpret_cast<float *>(smem + P.o_lut);
    int32_t *s_tab = reinterpret_cast<int32_t *>(smem + P.o_tab);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem + P.o_bar);
    volatile uint32_t *s_misc = reinterpret_cast<volatile uint32_t *>(s_bar + TB_COUNT);
    CopyDesc *s_desc = reinterpret_cast<CopyDesc *>(smem + P.o_desc);
    const uint32_t bar0 = smem_u32(s_bar);
#define TBAR(slot) (bar0 + 8u * (uint32_t)(slot))

    // ---- prologue, spread over the CTA ----
    if (threadIdx.x < 16) {
        const int c = threadIdx.x;
        const int mi = ((c >> 1) & 3) * 2 + (c & 1);
        const float mag = mi == 0 ? 0.f : (mi == 1 ? .5f : (float)(2 + (mi & 1)) * (float)(1 << (mi >> 1)) * 0.25f);
        s_lut[c] = (c & 8) ? -mag : mag;
    }
    if (threadIdx.x == 32) {
        for (int s = 0; s < TC_MAX_STAGES; ++s) {
            mbar_init(TBAR(TB_FULL + s), 1);
            mbar_init(TBAR(TB_EMPTY + s), 4 * H);                   // every (unit, quarter) task of the group
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(TBAR(TB_KREADY + x), 16);                      // 4 units x 4 quarters
            mbar_init(TBAR(TB_VREADY + x), 16);
            mbar_init(TBAR(TB_DQFULL + x), 1);
            mbar_init(TBAR(TB_DQFREE + x), 4);
        }
        for (int x = 0; x < 4; ++x) {
            mbar_init(TBAR(TB_KFREE + x), 1);
            mbar_init(TBAR(TB_PVDONE + x), 1);
            mbar_init(TBAR(TB_PREADY + x), 4);
        }
        s_misc[TM_ABORT] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(const_cast<uint32_t *>(&s_misc[TM_TMEM]))), "r"(P.tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    if (threadIdx.x == 0 && p.swz != 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_v)) : "memory");
    }
    const int cpg = 4 * p.ppg + 6;                                      // copies per group = per stage
    {
        const uint32_t page_b = (uint32_t)p.ps * H;
        const int c = (int)threadIdx.x - 64;
        if (c >= 0 && c < cpg) {
            CopyDesc d;
            d.src = nullptr; d.unit = 0; d.dst = 0; d.tbase = 0; d.tmul = 0; d.gi = 0; d.tok0 = 0;
            if (c < 4 * p.ppg) {
                const int pg = c >> 2, plane = c & 3;
                const uint32_t w = plane < 2 ? 32u : (plane == 2 ? 4u : 8u);
                d.src = plane == 0 ? p.k_base : (plane == 1 ? p.v_main : (plane == 2 ? p.v_scale : p.v_zp));
                d.unit = page_b * w;
                d.dst = (plane == 0 ? 0u : (plane == 1 ? (uint32_t)p.o_vm : (plane == 2 ? (uint32_t)p.o_vs : (uint32_t)p.o_vz))) + (uint32_t)pg * page_b * w;
                d.tbase = pg; d.tmul = p.ppg; d.tok0 = pg * p.ps;
                if (p.swz != 0 && plane < 2) d.gi |= (plane + 1) << 8;
            } else {
                const int gp = c - 4 * p.ppg;
                const bool on = gp < 2 || (k_out > 0 && (gp >= 4 || p.use_map));
                if (on) {
                    const uint32_t w = gp == 0 ? 128u : (gp == 4 ? 128u * p.nbi : (gp == 5 ? 128u * p.nb : 256u));
                    d.src = gp == 0 ? p.k_scale : (gp == 1 ? p.k_zp : (gp == 2 ? p.k_ms : (gp == 3 ? p.k_mc : (gp == 4 ? p.k_obmp : p.k_oval))));
                    d.unit = (uint32_t)H * w;
                    d.dst = (uint32_t)(gp == 0 ? p.o_ks : (gp == 1 ? p.o_kz : (gp == 2 ? p.o_ms : (gp == 3 ? p.o_mc : (gp == 4 ? p.o_bm : p.o_ov)))));
                    d.tbase = P.tab_pages; d.tmul = 1;
                }
            }
            s_desc[c] = d;
        }
        const int g0 = p.seg_group_base + t0 / 32;
        const int npages = (ntok + p.ps - 1) / p.ps;
        const int64_t pg0 = ((int64_t)g0 * 32) / p.ps;
        for (int i = threadIdx.x; i < npages; i += TC_THREADS) {
            int64_t pg = load_index(p.r2t, p.tbl64, (int64_t)b * p.r2t_sb + pg0 + i);
            if (pg < 0 || pg >= p.num_pages) { or_status(p.status, OMMX_ST_BAD_PAGE); pg = 0; }
            s_tab[i] = (int)pg;
        }
        for (int i = TC_THREADS - 1 - (int)threadIdx.x; i < ngroups; i += TC_THREADS) {
            int64_t sl = load_index(p.r2g, p.tbl64, (int64_t)b * p.r2g_sb + g0 + i);
            if (sl < 0 || sl >= p.num_slots) { or_status(p.status, OMMX_ST_BAD_GROUP); sl = 0; }
            s_tab[P.tab_pages + i] = (int)sl;
        }
        // query tables, rows = (kv head, padded query head), columns in tile position order:
        // s_q16 = fp16 of bf16(q * sm_scale) for the B tile, s_qraw = the raw bf16 query for the q.zp sums
        for (int idx = threadIdx.x; idx < H * GQAP * 128; idx += TC_THREADS) {
            const int row = idx >> 7, ch = idx & 127;                  // consecutive threads read consecutive channels
            const int h = row / GQAP, j = row - h * GQAP;
            uint16_t raw = 0, q16 = 0;
            if (j < gqa) {
                const __nv_bfloat16 v = p.q[(int64_t)b * p.q_sb + (int64_t)(h * gqa + j) * p.q_sh + ch];
                raw = __bfloat16_as_ushort(v);
                q16 = (uint16_t)f16_bits_sat(bf16_round_f32(__bfloat162float(v) * p.sm_scale));
            }
            s_qraw[row * 128 + tc_pos_of(ch)] = raw;
            s_q16[row * 128 + tc_pos_of(ch)] = q16;
        }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // Register budget per role (setmaxnreg, warpgroup granularity; the CTA was launched with 768 x 80): the softmax
    // warpgroup (warps 4..7) carries the per-block sums, everyone else needs little.  128 x 120 + 640 x 72 = 768 x 80.
    if (!(warp >= TC_W_SOFTMAX && warp < TC_W_SOFTMAX + 4)) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    const uint32_t tmem = s_misc[TM_TMEM];
    const uint32_t tm_dqk = tmem, tm_dpv = tmem + 2 * N_QK;
    const float LOG2E = 1.4426950408889634f;
    const int TS = H * 32;

    if (warp == TC_W_PRODUCER) {
        // =========================== producer: one group per stage ===========================
        for (int g = 0; g < ngroups; ++g) {
            const int s = g % NS;
            const uint32_t ph = (uint32_t)(g / NS) & 1u;
            if (!mbar_wait(TBAR(TB_EMPTY + s), ph ^ 1)) {
                if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); s_misc[TM_ABORT] = 1; }
                break;
            }
            uint32_t mine = 0;
            for (int c = lane; c < cpg; c += 32) {
                const CopyDesc d = s_desc[c];
                if (d.unit && 32 * g + d.tok0 < ntok) mine += d.unit;
            }
            const uint32_t total = __reduce_add_sync(0xFFFFFFFFu, mine);
            if (lane == 0) mbar_arrive_expect_tx(TBAR(TB_FULL + s), total);
            __syncwarp();
            const uint32_t sbase = smem_u32(s_stage + (size_t)s * p.stage_bytes);
            for (int c = lane; c < cpg; c += 32) {
                const CopyDesc d = s_desc[c];
                const int kind = d.gi >> 8;
                if (d.unit && 32 * g + d.tok0 < ntok) {
                    const int64_t idx = s_tab[d.tbase + g * d.tmul];
                    if (kind == 0) bulk_g2s(sbase + d.dst, d.src + idx * d.unit, d.unit, TBAR(TB_FULL + s));
                    else tma_2d_g2s(sbase + d.dst, kind == 1 ? &p.tmap_k : &p.tmap_v, 0, (int32_t)idx * p.rows_per_page, TBAR(TB_FULL + s));
                }
            }
        }
    } else if (warp == TC_W_MMA) {
        // =========================== MMA issue (one thread) ===========================
        constexpr uint32_t ID_QK = umma_idesc_f16(128, N_QK, 0, 0);
        constexpr uint32_t ID_PV = umma_idesc_f16(128, N_PV, 1, 1);
        const uint32_t a_k = smem_u32(s_ktile), a_v = smem_u32(s_vtile), a_bq = smem_u32(s_bq), a_pt = smem_u32(s_pt);
        bool dead = false;
        // Event driven: whichever of "logits of item qk" and "output of item pv" has its operands ready is issued
        // next, the output first (it frees the V tile and the P' tiles).  Probes do not block; the loop gives up
        // when nothing became ready for about a second of SM clock.
        int qk = 0, pv = 0;
        long long t_last = clock64();
        uint32_t idle = 0;
        while (pv < n_items) {
            bool did = false;
            if (pv < qk) {
                const int i = pv, x = i & 1, vb = i % P.nvb;
                if (mbar_test(TBAR(TB_PREADY + (i & 3)), (uint32_t)(i >> 2) & 1u) &&
                    mbar_test(TBAR(TB_VREADY + vb), (uint32_t)(i / P.nvb) & 1u)) {
                    tc_fence_after();
                    if (lane == 0) {
                        for (int ub = 0; ub < 4; ++ub) {
                            if (4 * i + ub >= n_units) break;
                            const int blk = ub + (NB8 ? 4 * (i & 1) : 0);
                            const bool first = i < (NB8 ? 2 : 1);
                            const uint32_t d = tm_dpv + blk * N_PV;
                            const uint32_t av = a_v + vb * TC_VTILE + ub * TC_UNIT_TILE;
                            const uint32_t bp = a_pt + (x * 4 + ub) * PT_BYTES;
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks)
                                umma_f16(d, umma_desc(av + ks * 256, 128, 512), umma_desc(bp + ks * 256, 128, 512), ID_PV, (first && ks == 0) ? 0u : 1u);
                        }
                        umma_commit(TBAR(TB_PVDONE + (i & 3)));
                    }
                    __syncwarp();
                    ++pv;
                    did = true;
                }
            }
            if (!did && qk < n_items) {
                const int i = qk, x = i & 1;
                if (mbar_test(TBAR(TB_KREADY + x), (uint32_t)(i >> 1) & 1u) &&
                    (i < 2 || mbar_test(TBAR(TB_DQFREE + x), (uint32_t)((i >> 1) - 1) & 1u))) {
                    tc_fence_after();
                    if (lane == 0) {
                        const int ksteps = k_out > 0 ? TC_KCHUNKS / 2 : 8;      // the residual positions exist only with outliers
#pragma unroll
                        for (int ks = 0; ks < TC_KCHUNKS / 2; ++ks)
                            if (ks < ksteps)
                                umma_f16(tm_dqk + x * N_QK, umma_desc(a_k + x * TC_KTILE + ks * 4096, 2048, 128),
                                         umma_desc(a_bq + x * BQ_BYTES + ks * 2 * (16 * N_QK), 16 * N_QK, 128), ID_QK, ks > 0 ? 1u : 0u);
                        umma_commit(TBAR(TB_DQFULL + x));
                        umma_commit(TBAR(TB_KFREE + (i & 3)));
                    }
                    __syncwarp();
                    ++qk;
                    did = true;
                }
            }
            if (did) { idle = 0; t_last = clock64(); continue; }
            // nothing to issue: park on the event most likely to come next, for a fraction of a microsecond at most
            if (pv < qk) mbar_try_wait_ns(TBAR(TB_PREADY + (pv & 3)), (uint32_t)(pv >> 2) & 1u, 128u);
            else mbar_try_wait_ns(TBAR(TB_KREADY + (qk & 1)), (uint32_t)(qk >> 1) & 1u, 128u);
            if ((++idle & 63u) == 0 && (clock64() - t_last > WAIT_LIMIT_CYCLES || s_misc[TM_ABORT] != 0)) { dead = true; break; }
        }
        if (dead && lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); s_misc[TM_ABORT] = 1; }
    } else if (warp >= TC_W_SOFTMAX && warp < TC_W_SOFTMAX + 4) {
        // =========================== softmax warps ===========================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 120;");
        const int w = warp & 3;                                       // unit in item = lane quarter of tensor memory
        const uint32_t lane_base = (uint32_t)(32 * w) << 16;
        // per accumulator block: reference maximum, per-lane sums of P, per-lane sums of P * V zero-point [scale group][head]
        constexpr int NBZ = NB8 ? 4 * GQAP : 1;                       // the second block's zero-point sums exist only with 8 blocks
        float m0[GQAP], l0[GQAP], m1[GQAP], l1[GQAP], z0[4 * GQAP], z1[NBZ];
#pragma unroll
        for (int j = 0; j < GQAP; ++j) { m0[j] = m1[j] = -INFINITY; l0[j] = l1[j] = 0.f; }
#pragma unroll
        for (int j = 0; j < 4 * GQAP; ++j) z0[j] = 0.f;
#pragma unroll
        for (int j = 0; j < NBZ; ++j) z1[j] = 0.f;
        bool dead = false;

        // A bounded wait that runs out raises the CTA's abort flag; the four warps look at the flag right after
        // each of their common barriers, so they always leave the loop together and no barrier is left waiting.
        auto give_up = [&]() { if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); s_misc[TM_ABORT] = 1; } };
        auto item_body = [&](const int i, float (&mref)[GQAP], float (&lsum)[GQAP], auto &zsum) {
            const int x = i & 1, u = 4 * i + w;
            const bool valid = u < n_units;
            const int g = valid ? u / H : 0;
            uint32_t raw[GQAP];
#pragma unroll
            for (int j = 0; j < GQAP; ++j) raw[j] = 0u;
            if (mbar_wait(TBAR(TB_DQFULL + x), (uint32_t)(i >> 1) & 1u)) {
                tc_fence_after();
                tmem_ld<GQAP>(tm_dqk + lane_base + x * N_QK + w * GQAP, raw);
                tc_fence_before();
            } else {
                give_up();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(TBAR(TB_DQFREE + x));
            const uint8_t *side = s_side + x * TC_SIDE_BYTES;
            float xs[GQAP], mloc[GQAP];
            const bool tok_ok = valid && (32 * g + lane < ntok);
            {
                const float *qz = reinterpret_cast<const float *>(side + TC_SIDE_QZ) + w * 32;
#pragma unroll
                for (int j = 0; j < GQAP; ++j) {
                    float v = fmaf(__uint_as_float(raw[j]), (float)(1 << (16 - TC_FBQ)), ((qz[j] + qz[8 + j]) + (qz[16 + j] + qz[24 + j])) * p.sm_scale);
                    if (p.logit_cap > 0.f) v = p.logit_cap * tanhf(v / p.logit_cap);
                    xs[j] = tok_ok ? v : -INFINITY;
                    mloc[j] = redux_max_f32(xs[j]);
                }
            }
            // does the reference maximum of this block have to move?
            bool need = false, blk_started = false;
            float corr[GQAP];
#pragma unroll
            for (int j = 0; j < GQAP; ++j) {
                need |= (mloc[j] - mref[j]) * LOG2E > TC_RESCALE_LOG2;   // -inf reference: true whenever mloc is finite
                blk_started |= (mref[j] != -INFINITY);
            }
            const bool rescale = need && blk_started && valid;
#pragma unroll
            for (int j = 0; j < GQAP; ++j) {
                const float target = need ? fmaxf(mref[j], mloc[j]) : mref[j];
                const float safe = target == -INFINITY ? 0.f : target;
                corr[j] = (mref[j] == -INFINITY) ? (need ? 0.f : 1.f) : fast_exp2((mref[j] - safe) * LOG2E);
                mref[j] = target;
            }
            // publish, then all four warps look at all four flags: a block's accumulator spans every lane quarter
            if (lane == 0) {
                s_misc[TM_NEED + x * 4 + w] = rescale ? 1u : 0u;
                if (rescale) {
#pragma unroll
                    for (int j = 0; j < GQAP; ++j) s_misc[TM_CORR + (x * 4 + w) * 8 + j] = __float_as_uint(corr[j]);
                }
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (s_misc[TM_ABORT] != 0) { dead = true; return; }
            uint32_t anyneed = 0;
#pragma unroll
            for (int o = 0; o < 4; ++o) anyneed |= s_misc[TM_NEED + x * 4 + o] << o;
            if (anyneed) {
                // every output MMA issued so far must have landed before its accumulator is rewritten
                const bool landed = i < 1 || mbar_wait(TBAR(TB_PVDONE + ((i - 1) & 3)), (uint32_t)((i - 1) >> 2) & 1u);
                if (!landed) give_up();
                tc_fence_after();
                if (landed) {
#pragma unroll
                    for (int o = 0; o < 4; ++o) {
                        if (!(anyneed & (1u << o))) continue;
                        const int blk = o + (NB8 ? 4 * (i & 1) : 0);
                        const uint32_t addr = tm_dpv + lane_base + blk * N_PV + w * GQAP;   // this quarter's scale-group columns
                        uint32_t acc[GQAP];
                        tmem_ld<GQAP>(addr, acc);
#pragma unroll
                        for (int j = 0; j < GQAP; ++j)
                            acc[j] = __float_as_uint(__uint_as_float(acc[j]) * __uint_as_float(s_misc[TM_CORR + (x * 4 + o) * 8 + j]));
                        tmem_st<GQAP>(addr, acc);
                    }
                }
                tc_fence_before();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (s_misc[TM_ABORT] != 0) { dead = true; return; }
            }
            // probabilities against the reference maximum; the unit's P' tile; its share of the V zero-point term
            float pr[GQAP];
#pragma unroll
            for (int j = 0; j < GQAP; ++j) {
                const float ms = mref[j] == -INFINITY ? 0.f : mref[j];
                pr[j] = fast_exp2((xs[j] - ms) * LOG2E);                 // masked tokens: exp2(-inf) = 0
                lsum[j] = lsum[j] * corr[j] + pr[j];
            }
            bool tiles_free = true;
            if (i >= 2) tiles_free = mbar_wait(TBAR(TB_PVDONE + ((i - 2) & 3)), (uint32_t)((i - 2) >> 2) & 1u);   // tiles of item i - 2 consumed
            if (!tiles_free) give_up();
            if (valid && tiles_free) {
                const uint2 vf = *reinterpret_cast<const uint2 *>(side + TC_SIDE_VF + (w * 32 + lane) * 8);
                const uint2 vz = *reinterpret_cast<const uint2 *>(side + TC_SIDE_VZ + (w * 32 + lane) * 8);
                const float vzf[4] = {bf16_bits_to_f32(vz.x & 0xFFFFu), bf16_bits_to_f32(vz.x >> 16), bf16_bits_to_f32(vz.y & 0xFFFFu), bf16_bits_to_f32(vz.y >> 16)};
#pragma unroll
                for (int cg = 0; cg < 4; ++cg)
#pragma unroll
                    for (int j = 0; j < GQAP; ++j) zsum[cg * GQAP + j] = fmaf(zsum[cg * GQAP + j], corr[j], pr[j] * vzf[cg]);
                uint32_t pp[GQAP / 2];
#pragma unroll
                for (int j = 0; j < GQAP / 2; ++j) pp[j] = pack_f16x2(pr[2 * j], pr[2 * j + 1]);
                const uint32_t f2[4] = {dup16(vf.x & 0xFFFFu), dup16(vf.x >> 16), dup16(vf.y & 0xFFFFu), dup16(vf.y >> 16)};
                uint8_t *dst = s_pt + (x * 4 + w) * PT_BYTES + 16 * lane;
                if constexpr (GQAP == 4) {
#pragma unroll
                    for (int nb2 = 0; nb2 < 2; ++nb2)                    // row block of 8 = two scale groups x four heads
                        *reinterpret_cast<uint4 *>(dst + nb2 * 512) =
                            make_uint4(hmul2_f16(pp[0], f2[2 * nb2]), hmul2_f16(pp[1], f2[2 * nb2]),
                                       hmul2_f16(pp[0], f2[2 * nb2 + 1]), hmul2_f16(pp[1], f2[2 * nb2 + 1]));
                } else {
#pragma unroll
                    for (int cg = 0; cg < 4; ++cg)                       // row block of 8 = one scale group x eight heads
                        *reinterpret_cast<uint4 *>(dst + cg * 512) =
                            make_uint4(hmul2_f16(pp[0], f2[cg]), hmul2_f16(pp[1], f2[cg]), hmul2_f16(pp[2], f2[cg]), hmul2_f16(pp[3], f2[cg]));
                }
            } else if (valid) {
#pragma unroll
                for (int j = 0; j < 4 * GQAP; ++j) zsum[j] *= corr[j % GQAP];
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(TBAR(TB_PREADY + (i & 3)));
        };

        for (int i = 0; i < n_items && !dead; ++i) {
            if constexpr (NB8) {
                if (!(i & 1)) item_body(i, m0, l0, z0);
                else item_body(i, m1, l1, z1);
            } else {
                item_body(i, m0, l0, z0);
            }
        }

        // ---- epilogue: block states to shared memory, then every warp finishes its 32 channel rows ----
#pragma unroll
        for (int j = 0; j < GQAP; ++j) {
            float a = l0[j], c = l1[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xFFFFFFFFu, a, o); c += __shfl_xor_sync(0xFFFFFFFFu, c, o); }
            if (lane == 0) {
                s_misc[TM_FM + w * 8 + j] = __float_as_uint(m0[j]); s_misc[TM_FL + w * 8 + j] = __float_as_uint(a);
                s_misc[TM_FM + (w + 4) * 8 + j] = __float_as_uint(m1[j]); s_misc[TM_FL + (w + 4) * 8 + j] = __float_as_uint(c);
            }
        }
#pragma unroll
        for (int j = 0; j < 4 * GQAP; ++j) {
            float a = z0[j], c = NB8 ? z1[NB8 ? j : 0] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xFFFFFFFFu, a, o); if (NB8) c += __shfl_xor_sync(0xFFFFFFFFu, c, o); }
            if (lane == 0) {
                s_misc[TM_FB + w * 32 + j] = __float_as_uint(a);
                if (NB8) s_misc[TM_FB + (w + 4) * 32 + j] = __float_as_uint(c);
            }
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        bool fin_ok = !dead && s_misc[TM_ABORT] == 0;
        if (fin_ok && n_items > 0) fin_ok = mbar_wait(TBAR(TB_PVDONE + ((n_items - 1) & 3)), (uint32_t)((n_items - 1) >> 2) & 1u);
        tc_fence_after();
        const int nbh = P.nb / H;                                        // accumulator blocks per kv head (1, 2 or 4)
        const int m_row = 32 * w + lane;                                 // tile row = tensor-memory lane
        const int ch = tc_channel_of(m_row);
        const float row_f = exp2f((float)(24 - 2 * tc_vslot(m_row) - TC_FBV));
        for (int h = 0; h < H; ++h) {
            float acc[GQAP], den[GQAP], mx[GQAP];
#pragma unroll
            for (int j = 0; j < GQAP; ++j) { acc[j] = 0.f; den[j] = 0.f; mx[j] = -INFINITY; }
            for (int r = 0; r < nbh; ++r) {
                const int blk = h + r * H;
                if (blk >= n_units) continue;
#pragma unroll
                for (int j = 0; j < GQAP; ++j) mx[j] = fmaxf(mx[j], __uint_as_float(s_misc[TM_FM + blk * 8 + j]));
            }
            for (int r = 0; r < nbh; ++r) {
                const int blk = h + r * H;
                if (blk >= n_units || !fin_ok) continue;
                uint32_t d[GQAP];
                tmem_ld<GQAP>(tm_dpv + lane_base + blk * N_PV + w * GQAP, d);
#pragma unroll
                for (int j = 0; j < GQAP; ++j) {
                    const float mb = __uint_as_float(s_misc[TM_FM + blk * 8 + j]);
                    const float wgt = (mb == -INFINITY) ? 0.f : fast_exp2((mb - mx[j]) * LOG2E);
                    acc[j] = fmaf(fmaf(__uint_as_float(d[j]), row_f, __uint_as_float(s_misc[TM_FB + blk * 32 + w * GQAP + j])), wgt, acc[j]);
                    den[j] = fmaf(__uint_as_float(s_misc[TM_FL + blk * 8 + j]), wgt, den[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < GQAP; ++j) {
                if (j >= gqa) continue;
                float *dst = p.al + (int64_t)b * p.al_sb + (int64_t)(h * gqa + j) * p.al_sh + (int64_t)split * p.al_ss;
                const bool some = fin_ok && den[j] > 0.f;
                dst[ch] = some ? acc[j] / den[j] : 0.f;
                if (w == 0 && lane == 0) dst[HD] = some ? mx[j] + logf(den[j]) : -INFINITY;
            }
        }
        tc_fence_before();
    } else {
        // =========================== decode warps ===========================
        // A task is (item, unit, channel quarter): 32 channels = two 32-bit code words per token, lane = token for the
        // code expansion and lane = channel for the outliers.  16 tasks per item, dealt round-robin.
        const int dw = warp < TC_W_SOFTMAX ? warp - 2 : warp - 6;        // 0..TC_NDW-1
        bool dead = false;
        for (int task = dw; task < n_items * 16 && !dead; task += TC_NDW) {
            const int i = task >> 4, ub = (task >> 2) & 3, qt = task & 3, x = i & 1;
            const int u = 4 * i + ub;
            const bool valid = u < n_units;
            const int g = valid ? u / H : 0, h = valid ? u - g * H : 0;
            const int s = g % NS;
            // Item i - 2 used the same K tile, B tile and factor buffers: its logits must have been computed and its
            // softmax must have read the factors.  These waits come first: they also mean that every earlier user of
            // this group's ring stage has long seen it filled, so the parity asked for below is the right phase.
            if (i >= 2 && !mbar_wait(TBAR(TB_KFREE + ((i - 2) & 3)), (uint32_t)((i - 2) >> 2) & 1u)) { dead = true; break; }
            if (i >= 2 && !mbar_wait(TBAR(TB_PREADY + ((i - 2) & 3)), (uint32_t)((i - 2) >> 2) & 1u)) { dead = true; break; }
            if (valid && !mbar_wait(TBAR(TB_FULL + s), (uint32_t)(g / NS) & 1u)) { dead = true; break; }
            const uint8_t *gb = s_stage + (size_t)s * p.stage_bytes;
            uint8_t *ktile = s_ktile + x * TC_KTILE;
            uint8_t *side = s_side + x * TC_SIDE_BYTES;
            bool clamped_any = false;
            if (valid) {
                // ---- K codes: token row `lane`, two 32-bit words = channels 32qt .. 32qt+31 -> four 8-position chunks ----
                {
                    const uint2 kw = *reinterpret_cast<const uint2 *>(gb + swz128((uint32_t)(lane * TS + h * 32 + 8 * qt), p.swz));
                    uint8_t *row = ktile + 16 * (32 * ub + lane) + (4 * qt) * 2048;
                    const uint32_t M = 0x03000300u;
                    *reinterpret_cast<uint4 *>(row) = make_uint4((kw.x << 8) & M, (kw.x << 6) & M, (kw.x << 4) & M, (kw.x << 2) & M);
                    *reinterpret_cast<uint4 *>(row + 2048) = make_uint4(kw.x & M, (kw.x >> 2) & M, (kw.x >> 4) & M, (kw.x >> 6) & M);
                    *reinterpret_cast<uint4 *>(row + 4096) = make_uint4((kw.y << 8) & M, (kw.y << 6) & M, (kw.y << 4) & M, (kw.y << 2) & M);
                    *reinterpret_cast<uint4 *>(row + 6144) = make_uint4(kw.y & M, (kw.y >> 2) & M, (kw.y >> 4) & M, (kw.y >> 6) & M);
                }
                // ---- B tile rows of this unit (query x 2^(e_k + FBQ)) and the fp32 q.zp sums of positions 32qt .. 32qt+31:
                //      lane = (8-position chunk c of 4, head j of 8) ----
                {
                    const int c = lane & 3, j = lane >> 2;
                    const int kc = 4 * qt + c;                                            // chunk of the row
                    const int c0 = 16 * (kc >> 1) + 4 * (kc & 1);                         // channels c0..c0+3 (even positions), c0+8.. (odd)
                    float sum = 0.f;
                    if (j < GQAP) {
                        const uint32_t ea = *reinterpret_cast<const uint32_t *>(gb + p.o_ks + h * 128 + c0);
                        const uint32_t eb = *reinterpret_cast<const uint32_t *>(gb + p.o_ks + h * 128 + c0 + 8);
                        uint32_t fac[4];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            bool c1, c2;
                            const uint32_t fa = tc_pow2_f16(max((int)(int8_t)(ea >> (8 * t)), -126), TC_FBQ, c1);
                            const uint32_t fb = tc_pow2_f16(max((int)(int8_t)(eb >> (8 * t)), -126), TC_FBQ, c2);
                            clamped_any |= c1 | c2;
                            fac[t] = fa | (fb << 16);
                        }
                        const uint2 za = *reinterpret_cast<const uint2 *>(gb + p.o_kz + h * 256 + 2 * c0);
                        const uint2 zb = *reinterpret_cast<const uint2 *>(gb + p.o_kz + h * 256 + 2 * (c0 + 8));
                        const int qrow = (h * GQAP + j) * 128 + 8 * kc;
                        const uint4 q = *reinterpret_cast<const uint4 *>(s_q16 + qrow);
                        *reinterpret_cast<uint4 *>(s_bq + x * BQ_BYTES + 16 * (ub * GQAP + j) + kc * (16 * N_QK)) =
                            make_uint4(hmul2_f16(q.x, fac[0]), hmul2_f16(q.y, fac[1]), hmul2_f16(q.z, fac[2]), hmul2_f16(q.w, fac[3]));
                        const uint4 r = *reinterpret_cast<const uint4 *>(s_qraw + qrow);
                        const uint32_t rw[4] = {r.x, r.y, r.z, r.w}, zaw[4] = {za.x & 0xFFFFu, za.x >> 16, za.y & 0xFFFFu, za.y >> 16},
                                       zbw[4] = {zb.x & 0xFFFFu, zb.x >> 16, zb.y & 0xFFFFu, zb.y >> 16};
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            sum = fmaf(bf16_bits_to_f32(rw[t] & 0xFFFFu), bf16_bits_to_f32(zaw[t]), fmaf(bf16_bits_to_f32(rw[t] >> 16), bf16_bits_to_f32(zbw[t]), sum));
                    }
                    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                    if (c == 0 && j < GQAP) reinterpret_cast<float *>(side + TC_SIDE_QZ)[ub * 32 + qt * 8 + j] = sum;
                }
                // ---- V factors of tokens 8qt .. 8qt+7: lane = (token, scale group) ----
                {
                    const int tk = 8 * qt + (lane & 7), cg = lane >> 3;
                    uint32_t fbits = 0u, zbits = 0u;
                    if (32 * g + tk < ntok) {
                        bool c1;
                        fbits = tc_pow2_f16((int)(int8_t)gb[p.o_vs + (tk * H + h) * 4 + cg], TC_FBV, c1, TC_VF_LIMIT);
                        clamped_any |= c1;
                        zbits = *reinterpret_cast<const uint16_t *>(gb + p.o_vz + (tk * H + h) * 8 + 2 * cg);   // bf16, as stored
                    }
                    *reinterpret_cast<uint16_t *>(side + TC_SIDE_VF + (ub * 32 + tk) * 8 + 2 * cg) = (uint16_t)fbits;
                    *reinterpret_cast<uint16_t *>(side + TC_SIDE_VZ + (ub * 32 + tk) * 8 + 2 * cg) = (uint16_t)zbits;
                }
                // ---- outliers of channel 32qt + lane, written over their slots of the K tile (after the codes) ----
                __syncwarp();
                if (k_out > 0) {
                    switch (k_out) {
                        case 2: tc_splice<2>(p, gb, ktile, s_bq + x * BQ_BYTES, s_q16, s_lut, h, ub, qt, lane, GQAP, N_QK, clamped_any); break;
                        case 4: tc_splice<4>(p, gb, ktile, s_bq + x * BQ_BYTES, s_q16, s_lut, h, ub, qt, lane, GQAP, N_QK, clamped_any); break;
                        case 6: tc_splice<6>(p, gb, ktile, s_bq + x * BQ_BYTES, s_q16, s_lut, h, ub, qt, lane, GQAP, N_QK, clamped_any); break;
                        case 8: tc_splice<8>(p, gb, ktile, s_bq + x * BQ_BYTES, s_q16, s_lut, h, ub, qt, lane, GQAP, N_QK, clamped_any); break;
                        default: tc_splice<-1>(p, gb, ktile, s_bq + x * BQ_BYTES, s_q16, s_lut, h, ub, qt, lane, GQAP, N_QK, clamped_any); break;
                    }
                }
            }
            if (clamped_any) or_status(p.status, OMMX_ST_SCALE_RANGE);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(TBAR(TB_KREADY + x));

            // ---- V codes of this quarter into the V tile (channel-major), once the tile's previous user is done ----
            const int vb = i % P.nvb;
            if (i >= P.nvb) {
                const int jdone = i - P.nvb;
                if (!mbar_wait(TBAR(TB_PVDONE + (jdone & 3)), (uint32_t)(jdone >> 2) & 1u)) { dead = true; break; }
            }
            if (valid) {
                uint2 vw = make_uint2(0u, 0u);
                if (32 * g + lane < ntok) vw = *reinterpret_cast<const uint2 *>(gb + p.o_vm + swz128((uint32_t)(lane * TS + h * 32 + 8 * qt), p.swz));
                uint8_t *vt = s_vtile + vb * TC_VTILE + ub * TC_UNIT_TILE + 16 * lane + (4 * qt) * 512;
                *reinterpret_cast<uint4 *>(vt) = make_uint4(code_pair(vw.x, 0), code_pair(vw.x, 1), code_pair(vw.x, 2), code_pair(vw.x, 3));
                *reinterpret_cast<uint4 *>(vt + 512) = make_uint4(code_pair(vw.x, 4), code_pair(vw.x, 5), code_pair(vw.x, 6), code_pair(vw.x, 7));
                *reinterpret_cast<uint4 *>(vt + 1024) = make_uint4(code_pair(vw.y, 0), code_pair(vw.y, 1), code_pair(vw.y, 2), code_pair(vw.y, 3));
                *reinterpret_cast<uint4 *>(vt + 1536) = make_uint4(code_pair(vw.y, 4), code_pair(vw.y, 5), code_pair(vw.y, 6), code_pair(vw.y, 7));
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(TBAR(TB_VREADY + vb));
                if (valid) mbar_arrive(TBAR(TB_EMPTY + s));
            }
        }
        if (dead && lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); s_misc[TM_ABORT] = 1; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TC_W_MMA) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(P.tmem_cols));
#undef TBAR
}

// ---- host side ----------------------------------------------------------------------------------
// Fills the tensor-core kernel's shared-memory layout; returns the bytes needed (0 = the shape is not served).
static size_t tc_layout(TcParams &P, int gqap, int max_groups_per_split) {
    S1Params &p = P.s;
    const int H = p.H;
    const int n_qk = 4 * gqap;
    const size_t bq = (size_t)TC_KCHUNKS * 16 * n_qk, pt = (size_t)(4 * gqap) * 64;
    P.nb = H > 4 ? H : 4;
    P.tab_groups = max_groups_per_split;
    P.tab_pages = max_groups_per_split * p.ppg;
    const size_t fixed = 2 * TC_KTILE + 2 * bq + 2 * 4 * pt + 2 * TC_SIDE_BYTES + 2 * (size_t)H * gqap * 256 + 64 +
                         (size_t)(P.tab_pages + P.tab_groups) * 4 + 64 + TB_COUNT * 8 + TM_WORDS * 4 + 64 +
                         (size_t)(4 * p.ppg + 6) * sizeof(CopyDesc) + 1024 /* alignment slack */ + 1024 /* offset rounding */;
    const size_t limit = 232448;
    const int min_stages = 2 * (H >= 4 ? 1 : 4 / H);                      // two items' worth of groups in flight
    int best_ns = 0, best_nvb = 0;
    for (int nvb = 2; nvb >= 1 && !best_ns; --nvb)
        for (int ns = TC_MAX_STAGES; ns >= min_stages; --ns)
            if (fixed + (size_t)nvb * TC_VTILE + (size_t)ns * p.stage_bytes <= limit) {
                // prefer the second V buffer only when at least 3 stages still fit
                if (nvb == 2 && ns < 3 && min_stages < 3) continue;
                best_ns = ns; best_nvb = nvb;
                break;
            }
    if (!best_ns) return 0;
    p.nstages = best_ns;
    P.nvb = best_nvb;
    auto up = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
    size_t o = (size_t)best_ns * p.stage_bytes;
    o = up(o, 128); P.o_ktile = (uint32_t)o; o += 2 * TC_KTILE;
    P.o_vtile = (uint32_t)o; o += (size_t)best_nvb * TC_VTILE;
    P.o_bq = (uint32_t)o; o += 2 * bq;
    P.o_ptile = (uint32_t)o; o += 2 * 4 * pt;
    P.o_side = (uint32_t)o; o += 2 * TC_SIDE_BYTES;
    P.o_q16 = (uint32_t)o; o += (size_t)H * gqap * 256;
    P.o_qraw = (uint32_t)o; o += (size_t)H * gqap * 256;
    P.o_lut = (uint32_t)o; o += 64;
    P.o_tab = (uint32_t)o; o += (size_t)(P.tab_pages + P.tab_groups) * 4;
    o = up(o, 16); P.o_bar = (uint32_t)o; o += TB_COUNT * 8 + TM_WORDS * 4;
    o = up(o, 16); P.o_desc = (uint32_t)o; o += (size_t)(4 * p.ppg + 6) * sizeof(CopyDesc);
    const int cols = 2 * n_qk + P.nb * (4 * gqap);
    P.tmem_cols = cols <= 32 ? 32 : (cols <= 64 ? 64 : (cols <= 128 ? 128 : (cols <= 256 ? 256 : 512)));
    if (cols > 512) return 0;
    return o + 1024;
}

template <int GQAP, bool NB8>
static int launch_tc(const TcParams &P, dim3 grid, size_t smem, cudaStream_t st) {
    static std::atomic<size_t> attr_smem[MAX_DEVICES];
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    if (smem > attr_smem[dev].load(std::memory_order_acquire)) {
        OMMX_CUDA_TRY(cudaFuncSetAttribute(decode_stage1_tc_kernel<GQAP, NB8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem[dev].store(smem, std::memory_order_release);
    }
    static std::atomic<int> regs_state[MAX_DEVICES];   // 0 unknown, 1 enough, 2 too few
    int regs_ok = regs_state[dev].load(std::memory_order_acquire);
    if (regs_ok == 0) {
        cudaFuncAttributes fa;
        OMMX_CUDA_TRY(cudaFuncGetAttributes(&fa, decode_stage1_tc_kernel<GQAP, NB8>));
        regs_ok = fa.numRegs * TC_THREADS >= 128 * 120 + (TC_THREADS - 128) * 72 ? 1 : 2;   // setmaxnreg.inc must find the registers
        regs_state[dev].store(regs_ok, std::memory_order_release);
    }
    if (regs_ok != 1) return fail(OMMX_E_CUDA, "the tensor-core stage 1 was compiled with fewer registers than its warp roles need");
    OMMX_CUDA_TRY(launch_overlapping_previous(decode_stage1_tc_kernel<GQAP, NB8>, grid, TC_THREADS, smem, st, P));
    count_launch();
    return 0;
}

}  // namespace ommx
