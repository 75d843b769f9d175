// Paged decode attention over OMMX-quantized KV planes for sm_100a: split-KV stage 1, stage 2
// (log-sum-exp combine with the bf16 sink/recent rows fused in) and the partial-state merge.
//
// Stage 1 replaces _canonical_splitkv_stage1 (ommx_gpu_serve/attention/paged_decode.py:1255-2284
// of the reference).  One CTA serves one (split, sequence) pair and ALL local kv heads of its
// token range, so every page row it touches is a full contiguous line:
//
//   producer warp   streams whole pages / group-slot planes into a 4-stage shared-memory ring
//                   with 1-D bulk async copies (cp.async.bulk + mbarrier transaction counts);
//                   page ids and group slots of the split are prefetched into shared memory once.
//   8 consumer warps each own one (group, kv head) unit per stage and keep a private online-
//                   softmax state.  Per unit:
//     phase A (lane = 4 channels): walk the outlier bitmask with clz, decode the FP4 nibble,
//                   and write the delta between the outlier value and the base code it replaces,
//                   expressed in code units, into a per-warp bf16 tile [token][channel-slot].
//     phase B (mma lanes): 2-bit codes -> bf16 with one LOP3 per pair (magic exponent, value
//                   128 + code*4^p), per-channel power-of-two scale folded into q, QK^T on
//                   mma.sync m16n8k16 (GQA rows padded to 16); the outlier tile is a second B
//                   operand read with ldmatrix; one extra tile row carries zp/scale and one
//                   carries -128, so q.zp and the magic offset come out of the same MMAs.
//                   Online softmax with quad shuffles, P in bf16, V dequantized in bf16x2
//                   (code*vs+vz, as the reference) and P.V on the same MMA shape.
//
// Numerics follow the reference kernel's rounding points: q*sm_scale rounded to bf16, exact
// code*2^e products, the outlier delta rounded to bf16, fp32 accumulation, P rounded to bf16, V
// dequantized to bf16.  One point differs at the bf16-rounding level: q.zp uses the bf16
// q*sm_scale instead of fp32 q.
#include "ommx_common.cuh"
#include <cuda.h>                       // CUtensorMap (types only; the encoder is looked up at run time)
#include <mutex>

namespace ommx {

constexpr int HD = 128;                 // head_dim this build serves
constexpr int NCW = 8;                  // (group, head) units in flight per CTA: 8 MMA warps + 8 decode warps
constexpr int NDW = 11;                 // decode warps (stateless tile builders, items dealt round-robin)
constexpr int PRODUCER_WARP = NCW + NDW;  // warp 19 streams the planes
constexpr int S1_THREADS = (NCW + NDW + 1) * 32;
// Register budget per role (setmaxnreg, warpgroup granularity).  Only what the CTA was launched with
// can be moved around: 640 threads x 96 = 61440 >= 256*152 (MMA) + 384*56 (decode + producer) = 60416.
#define OMMX_REGS_MMA "152"
#define OMMX_REGS_DECODE "56"
constexpr int NSTAGES = 4;
constexpr int DT_STRIDE = 272;          // bytes per outlier-tile row (256 data + 16 pad)
constexpr int DT_ROWS = 34;             // 32 tokens + zp row + (-128) row
constexpr int DT_BYTES = DT_ROWS * DT_STRIDE;
constexpr int MAX_SPLIT_GROUPS = 512;   // groups one CTA can index (16K tokens per split)
constexpr int MAX_SPLIT_PAGES = 2048;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;   // about a second of SM clock: the wait has failed

struct S1Params {
    const __nv_bfloat16 *q;
    int64_t q_sb, q_sh;
    int32_t B, Hq, H, gqa;
    const uint8_t *k_base, *v_main, *v_scale, *v_zp, *k_scale, *k_zp, *k_ms, *k_mc, *k_obmp, *k_oval;
    int32_t ps, ppg, num_pages, num_slots, k_out, nb, use_map;
    const int32_t *b_seq_len;
    const void *r2t, *r2g;
    int32_t tbl64;
    int64_t r2t_sb, r2g_sb;
    float *al;
    int64_t al_sb, al_sh, al_ss;
    int32_t S, seg_group_base;
    float sm_scale, logit_cap;
    int32_t *status;
    int32_t abl;
    // shared-memory layout of one group block (bytes)
    int32_t GS, gb_bytes, stage_bytes;
    int32_t o_vm, o_vs, o_vz, o_ks, o_kz, o_ms, o_mc, o_bm, o_ov;
    // tensor maps of the two code planes as [bytes/128][128] uint8 with 128-byte swizzle
    uint32_t swz;                        // 0x70 when the maps are in use, else 0
    int32_t rows_per_page;               // 128-byte lines per page
    alignas(64) CUtensorMap tmap_k;
    alignas(64) CUtensorMap tmap_v;
};

// One bulk copy of a stage: source plane, bytes, destination inside the stage, and which table entry
// (page id or group slot) selects the source block.
struct __align__(16) CopyDesc {
    const uint8_t *src;                  // plane base, or nullptr + kind for a tensor-map copy
    uint32_t unit, dst;
    int32_t tbase, tmul, gi, tok0;       // gi: group in stage (bits 0..7) | kind << 8
};                                       // kind 0 bulk copy, 1 k_base through tmap_k, 2 v_main through tmap_v
constexpr int MAX_STAGE_COPIES = 8 * (4 * 4 + 6);                    // 8 groups per stage, 8-token pages

// Development builds (-DOMMX_TRACE) stamp the SM clock at fixed points of one CTA's warps into a
// device array that ommx_b200_debug_read_trace copies out; service builds compile the probes away.
#ifdef OMMX_TRACE
__device__ long long g_trace[32 * 256];
#define OMMX_TR(slot)                                                                              \
    do {                                                                                           \
        if (blockIdx.x == 1 && blockIdx.y == 0 && lane == 0 && (slot) < 256) g_trace[warp * 256 + (slot)] = clock64(); \
    } while (0)
#else
#define OMMX_TR(slot) do { } while (0)
#endif

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and the caller raises OMMX_ST_TIMEOUT) instead of spinning forever.
// try_wait already parks the warp in hardware for a short while.  The limit is counted on the SM
// clock (cheap to read); nanosleep or the global timer in this loop would put their own latency
// on every producer/consumer hand-off.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const long long t_end = clock64() + WAIT_LIMIT_CYCLES;
#pragma unroll 1
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0 && clock64() > t_end) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The 2-bit code planes are staged with the TMA's 128-byte swizzle (16-byte chunk index XOR line
// index mod 8) when a page is a whole number of 1 KB swizzle atoms: a head's 32-byte code row then
// lands in a different bank window on each token row instead of the same one.  `o` is the linear byte
// offset inside a 1 KB aligned region; swz is 0x70 (swizzled) or 0 (plain bulk copies).
__device__ __forceinline__ uint32_t swz128(uint32_t o, uint32_t swz) { return o ^ ((o >> 3) & swz); }

__device__ __forceinline__ void tma_2d_g2s(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// position class of channel-in-word index i (0..7): the 2-bit field sits at bit 2*pc of its half
// when the LOP3 extracts it, so the extracted bf16 is 128 + code * 4^pc.
__device__ __forceinline__ int pos_class(int i) { return i < 3 ? i : (i < 6 ? i - 3 : i - 6); }

__device__ __forceinline__ int64_t load_index(const void *tbl, int is64, int64_t i) {
    return is64 ? reinterpret_cast<const int64_t *>(tbl)[i] : (int64_t) reinterpret_cast<const int32_t *>(tbl)[i];
}

// Extract the 8 bf16x2 registers of one 32-bit code word: register i holds (code i, code i+8)
// as bf16 values 128 + code * 4^pos_class(i).
__device__ __forceinline__ void codes_to_bf16x2(uint32_t w, uint32_t (&r)[8]) {
    const uint32_t M = 0x43004300u;
    r[0] = lop3_and_or(w, 0x00030003u, M);
    r[1] = lop3_and_or(w, 0x000C000Cu, M);
    r[2] = lop3_and_or(w, 0x00300030u, M);
    uint32_t t = w >> 6;
    r[3] = lop3_and_or(t, 0x00030003u, M);
    r[4] = lop3_and_or(t, 0x000C000Cu, M);
    r[5] = lop3_and_or(t, 0x00300030u, M);
    t = w >> 12;
    r[6] = lop3_and_or(t, 0x00030003u, M);
    r[7] = lop3_and_or(t, 0x000C000Cu, M);
}

// The same extraction in two halves (registers 0..3, then 4..7), for loops that interleave several
// code words so that back-to-back MMAs never share an accumulator.
__device__ __forceinline__ void codes_to_bf16x2_lo(uint32_t w, uint32_t (&r)[4]) {
    const uint32_t M = 0x43004300u;
    r[0] = lop3_and_or(w, 0x00030003u, M);
    r[1] = lop3_and_or(w, 0x000C000Cu, M);
    r[2] = lop3_and_or(w, 0x00300030u, M);
    r[3] = lop3_and_or(w >> 6, 0x00030003u, M);
}
__device__ __forceinline__ void codes_to_bf16x2_hi(uint32_t w, uint32_t (&r)[4]) {
    const uint32_t M = 0x43004300u;
    uint32_t t = w >> 6;
    r[0] = lop3_and_or(t, 0x000C000Cu, M);
    r[1] = lop3_and_or(t, 0x00300030u, M);
    t = w >> 12;
    r[2] = lop3_and_or(t, 0x00030003u, M);
    r[3] = lop3_and_or(t, 0x000C000Cu, M);
}

// =================================================================================================
// Stage 1
// =================================================================================================
// Ablation bits (differential timing only, they break parity; mirror of the reference's
// OMMX_ABL_* knobs, paged_decode.py:3267-3279): 1 = skip the outlier splice, 2 = skip V dequant
// and P.V, 4 = skip the K code dequant and its MMAs.
constexpr int ABL_NO_OUTLIER = 1, ABL_NO_V = 2, ABL_NO_K = 4, ABL_NO_COMPUTE = 8;   // 8: stream the planes only

// KOUT: outliers per K vector known at compile time (static, unrolled splice) or -1 (runtime).
// VFOLD: GQA groups of at most 4 query heads.  The 16 MMA rows are (query head, V scale group)
//        pairs, the per-(token, group) power-of-two V scale is folded into P, and V enters the
//        MMA as raw 128 + code*4^pc values: no per-element V arithmetic at all.  The offset comes
//        back out through a row-sum column, the zero-points through a small bias MMA.
template <int KOUT, bool VFOLD>
__global__ void __launch_bounds__(S1_THREADS, 1) decode_stage1_kernel(const __grid_constant__ S1Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // swizzle atoms are 1 KB: align the ring by hand (the launch adds 1 KB of slack)
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int split = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    OMMX_TR(250);

    // ---- split range (same rounding as the reference, paged_decode.py:1428-1432) ----
    const int seq = p.b_seq_len[b];
    if (seq <= 0) return;
    const int per = (((seq + p.S - 1) / p.S) + 31) / 32 * 32;
    const int t0 = split * per;
    const int t1 = min(t0 + per, seq);
    if (t1 <= t0) return;
    const int ntok = t1 - t0;
    int ngroups = (ntok + 31) / 32;
    if (ngroups > MAX_SPLIT_GROUPS) {                 // host sizing should prevent this
        if (threadIdx.x == 0) or_status(p.status, OMMX_ST_BAD_LENGTH);
        return;
    }
    const int H = p.H, GS = p.GS;
    const int n_iters = (ngroups + GS - 1) / GS;
    const int k_out = KOUT >= 0 ? KOUT : p.k_out;

    // ---- shared memory carve-up ----
    uint8_t *s_stage = smem;                                            // NSTAGES * stage_bytes
    uint8_t *s_tiles = s_stage + NSTAGES * p.stage_bytes;               // NCW * DT_BYTES
    int32_t *s_tab = reinterpret_cast<int32_t *>(s_tiles + NCW * DT_BYTES);   // page ids, then group slots
    float *s_lut = reinterpret_cast<float *>(s_tab + MAX_SPLIT_PAGES + MAX_SPLIT_GROUPS);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(s_lut + 16);         // full[NSTAGES], empty[NSTAGES], tile_full[NCW], tile_empty[NCW][NSTAGES]
    int32_t *s_abort = reinterpret_cast<int32_t *>(s_bar + 2 * NSTAGES + (1 + NSTAGES) * NCW);
    CopyDesc *s_desc = reinterpret_cast<CopyDesc *>(s_abort + 4);
    const uint32_t bar_full = smem_u32(s_bar), bar_empty = smem_u32(s_bar + NSTAGES);
    const uint32_t bar_tfull = smem_u32(s_bar + 2 * NSTAGES), bar_tempty = smem_u32(s_bar + 2 * NSTAGES + NCW);

    // ---- prologue: LUT, barriers, copy descriptors and the split's page / slot tables, spread over the
    //      whole CTA so that the producer can issue the first stage right after the barrier ----
    if (threadIdx.x < 16) {
        const int c = threadIdx.x;
        const int mi = ((c >> 1) & 3) * 2 + (c & 1);                    // exp*2 + mant
        const float mag = mi == 0 ? 0.f : (mi == 1 ? .5f : (float)(2 + (mi & 1)) * (float)(1 << (mi >> 1)) * 0.25f);
        s_lut[c] = (c & 8) ? -mag : mag;
    }
    if (threadIdx.x == 32) {
        for (int s = 0; s < NSTAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 2 * NCW);
        }
        for (int u = 0; u < NCW; ++u) {
            mbar_init(bar_tfull + 8 * u, 1);
            for (int k2 = 0; k2 < NSTAGES; ++k2) mbar_init(bar_tempty + 8 * (NSTAGES * u + k2), 1);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int cpg = 4 * p.ppg + 6;                                      // copies per group
    const int ncopies = GS * cpg;
    {
        // Copy roles (group-in-stage, plane) are tabulated once; the producer's loop body is then one
        // descriptor load, one table lookup, one multiply-add and one copy per role, with no divergent
        // paths, because that single warp's issue latency bounds how fast stages refill.
        const uint32_t page_b = (uint32_t)p.ps * H;                     // (token, head) rows per page
        const int c = (int)threadIdx.x - 64;                            // threads 64.. build one descriptor each
        if (c >= 0 && c < ncopies) {
            CopyDesc d;
            d.src = nullptr; d.unit = 0; d.dst = 0; d.tbase = 0; d.tmul = 0; d.gi = 0; d.tok0 = 0;
            const int gi = c / cpg, ci = c - gi * cpg;
            d.gi = gi;
            const uint32_t gbo = (uint32_t)gi * p.gb_bytes;
            if (ci < 4 * p.ppg) {
                const int pg = ci >> 2, plane = ci & 3;
                const uint32_t w = plane < 2 ? 32u : (plane == 2 ? 4u : 8u);
                d.src = plane == 0 ? p.k_base : (plane == 1 ? p.v_main : (plane == 2 ? p.v_scale : p.v_zp));
                d.unit = page_b * w;
                d.dst = gbo + (plane == 0 ? 0u : (plane == 1 ? (uint32_t)p.o_vm : (plane == 2 ? (uint32_t)p.o_vs : (uint32_t)p.o_vz)))
                      + (uint32_t)pg * page_b * w;
                d.tbase = pg; d.tmul = p.ppg; d.tok0 = pg * p.ps;
                if (p.swz != 0 && plane < 2) d.gi |= (plane + 1) << 8;
            } else {
                const int gp = ci - 4 * p.ppg;
                const bool on = gp < 2 || (k_out > 0 && (gp >= 4 || p.use_map));
                if (on) {
                    const uint32_t w = gp == 0 ? 128u : (gp == 4 ? 512u : (gp == 5 ? 128u * p.nb : 256u));
                    d.src = gp == 0 ? p.k_scale : (gp == 1 ? p.k_zp : (gp == 2 ? p.k_ms : (gp == 3 ? p.k_mc : (gp == 4 ? p.k_obmp : p.k_oval))));
                    d.unit = (uint32_t)H * w;
                    d.dst = gbo + (uint32_t)(gp == 0 ? p.o_ks : (gp == 1 ? p.o_kz : (gp == 2 ? p.o_ms : (gp == 3 ? p.o_mc : (gp == 4 ? p.o_bm : p.o_ov)))));
                    d.tbase = MAX_SPLIT_PAGES; d.tmul = 1;
                }
            }
            s_desc[c] = d;
        }
        // page ids first (s_tab[0..)), group slots behind them
        const int g0 = p.seg_group_base + t0 / 32;                      // first logical group
        const int npages = (ntok + p.ps - 1) / p.ps;
        const int64_t pg0 = ((int64_t)g0 * 32) / p.ps;
        for (int i = threadIdx.x; i < npages; i += S1_THREADS) {
            int64_t pg = load_index(p.r2t, p.tbl64, (int64_t)b * p.r2t_sb + pg0 + i);
            if (pg < 0 || pg >= p.num_pages) { or_status(p.status, OMMX_ST_BAD_PAGE); pg = 0; }
            s_tab[i] = (int)pg;
        }
        for (int i = S1_THREADS - 1 - (int)threadIdx.x; i < ngroups; i += S1_THREADS) {
            int64_t sl = load_index(p.r2g, p.tbl64, (int64_t)b * p.r2g_sb + g0 + i);
            if (sl < 0 || sl >= p.num_slots) { or_status(p.status, OMMX_ST_BAD_GROUP); sl = 0; }
            s_tab[MAX_SPLIT_PAGES + i] = (int)sl;
        }
    }
    __syncthreads();
    OMMX_TR(251);
    // Stage 2 is launched as a programmatic dependent: it may start its own prologue (residual-row
    // logits, which do not depend on this kernel) as soon as SM resources free up, and waits for this
    // grid to finish before it reads the split partials.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- roles; each branch starts by resizing its warpgroups' register budget and never rejoins ----
    if (warp >= NCW) asm volatile("setmaxnreg.dec.sync.aligned.u32 " OMMX_REGS_DECODE ";");
    if (warp == PRODUCER_WARP) {
        // =========================== producer warp ===========================
        uint32_t full_total = 0;                                        // bytes of a stage with GS whole groups
        for (int c = lane; c < ncopies; c += 32) full_total += s_desc[c].unit;
        full_total = __reduce_add_sync(0xFFFFFFFFu, full_total);
        const int whole_groups = ntok / 32;
        for (int it = 0; it < n_iters; ++it) {
            const int s = it % NSTAGES;
            const uint32_t ph = (it / NSTAGES) & 1;
            OMMX_TR(4 * it);
            if (!mbar_wait(bar_empty + 8 * s, ph ^ 1)) {
                if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                break;
            }
            OMMX_TR(4 * it + 1);
            const int lg0 = it * GS;
            uint32_t total = full_total;
            if (lg0 + GS > whole_groups) {                              // last stage: fewer groups or a partial group
                uint32_t mine = 0;
                for (int c = lane; c < ncopies; c += 32) {
                    const CopyDesc d = s_desc[c];
                    const int lg = lg0 + (d.gi & 0xFF);
                    if (d.unit && lg < ngroups && 32 * lg + d.tok0 < ntok) mine += d.unit;
                }
                total = __reduce_add_sync(0xFFFFFFFFu, mine);
            }
            if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * s, total);
            __syncwarp();
            const uint32_t sbase = smem_u32(s_stage + (size_t)s * p.stage_bytes);
            for (int c = lane; c < ncopies; c += 32) {
                const CopyDesc d = s_desc[c];
                const int lg = lg0 + (d.gi & 0xFF);
                const int kind = d.gi >> 8;
                if (d.unit && lg < ngroups && 32 * lg + d.tok0 < ntok) {
                    const int64_t idx = s_tab[d.tbase + lg * d.tmul];
                    if (kind == 0) bulk_g2s(sbase + d.dst, d.src + idx * d.unit, d.unit, bar_full + 8 * s);
                    else tma_2d_g2s(sbase + d.dst, kind == 1 ? &p.tmap_k : &p.tmap_v, 0, (int32_t)idx * p.rows_per_page, bar_full + 8 * s);
                }
            }
            OMMX_TR(4 * it + 2);
        }
        // fall through to the two CTA-wide barriers of the epilogue
        __syncthreads();
        __syncthreads();
        return;
    }

    // =========================== decode + MMA warps ===========================
    // MMA warp w owns unit w = (group-in-stage, kv head) and its softmax state.  The decode warps are
    // stateless: work item (iteration, unit) number n goes to decode warp n % NDW.
    const int g = lane >> 2, j = lane & 3;
    const int TS = H * 32;                                          // bytes per token row (all heads)
    const float LOG2E = 1.4426950408889634f;
    const bool no_outlier = (p.abl & ABL_NO_OUTLIER) != 0;

    if (warp >= NCW) {
        // =========================== decode warps (phase A) ===========================
        // Build a unit's outlier-delta tile one group ahead of its MMA warp: wait until the MMA warp
        // has read the previous tile of that unit, write the new one, publish it.
        const int dw = warp - NCW;
        // this lane owns channels 4*lane + c
        uint32_t pa_col[4];       // byte offset of the channel's column inside an outlier-tile row
        float pa_f[4];            // 4^pc of the channel's slot
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int d = 4 * lane + c;
            const int jj = d >> 5, wi = (d >> 4) & 1, i = d & 7, hi = (d >> 3) & 1;
            pa_col[c] = 2u * (16 * (4 * wi + (i >> 1)) + 8 * (i & 1) + 2 * jj + hi);
            pa_f[c] = (float)(1 << (2 * pos_class(i)));
        }
        if (dw < NCW) {           // item (0, dw) is this warp's: it is the first to touch tile dw
            uint8_t *t0p = s_tiles + dw * DT_BYTES;
            // row 33 = -128 in every column (never rewritten); clear the rest once
            for (int i = lane; i < DT_BYTES / 4; i += 32) reinterpret_cast<uint32_t *>(t0p)[i] = 0u;
            __syncwarp();
            for (int i = lane; i < 64; i += 32) reinterpret_cast<uint32_t *>(t0p + 33 * DT_STRIDE)[i] = 0xC300C300u;
            __syncwarp();
        }
        for (int n = dw; n < n_iters * NCW; n += NDW) {
            const int it = n / NCW, unit = n % NCW;
            const int trk = 8 * ((n - dw) / NDW);
            OMMX_TR(trk);
            const int h = unit % H, gsel = unit / H;
            uint8_t *tile = s_tiles + unit * DT_BYTES;
            const int s = it % NSTAGES;
            const uint32_t ph = (it / NSTAGES) & 1;
            if (!mbar_wait(bar_full + 8 * s, ph)) {
                if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                break;
            }
            OMMX_TR(trk + 1);
            const int lg = it * GS + gsel;                           // local group of this unit
            if (lg < ngroups && !(p.abl & ABL_NO_COMPUTE)) {
                // Tile `it` of a unit may be written once the MMA warp has read tile it-1.  Decode warps
                // run up to NSTAGES groups ahead and the tiles of one unit are built by different warps,
                // so "tile k was read" events rotate over NSTAGES barriers per unit (barrier k % NSTAGES,
                // phase k / NSTAGES): the newest event a waiter can be missing is then always the one it
                // waits for, never an older phase of the same parity.
                uint8_t *gb = s_stage + (size_t)s * p.stage_bytes + (size_t)gsel * p.gb_bytes;
                const uint8_t *ksc = gb + p.o_ks + h * 128;
                const uint8_t *kzp = gb + p.o_kz + h * 256;
                if (it > 0 && !mbar_wait(bar_tempty + 8 * (NSTAGES * unit + ((it - 1) % NSTAGES)),
                                         (uint32_t)((it - 1) / NSTAGES) & 1u)) {
                    if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                    break;
                }
                OMMX_TR(trk + 2);
            {
                    const bool splice = k_out > 0 && !no_outlier;
                    if (splice) {
                        // clear token rows 0..31 (256 data bytes each)
#pragma unroll
                        for (int r2 = 0; r2 < 16; ++r2)
                            *reinterpret_cast<uint4 *>(tile + (2 * r2 + (lane >> 4)) * DT_STRIDE + (lane & 15) * 16) = make_uint4(0, 0, 0, 0);
                        __syncwarp();
                    }
                    const uint32_t e4 = *reinterpret_cast<const uint32_t *>(ksc + 4 * lane);
                    const uint2 z4 = *reinterpret_cast<const uint2 *>(kzp + 8 * lane);
                    uint2 ms4 = make_uint2(0, 0), mc4 = make_uint2(0, 0);
                    uint4 bm4 = make_uint4(0, 0, 0, 0);
                    uint32_t st[4] = {0, 0, 0, 0};
                    if (splice) {
                        if (p.use_map) {
                            ms4 = *reinterpret_cast<const uint2 *>(gb + p.o_ms + h * 256 + 8 * lane);
                            mc4 = *reinterpret_cast<const uint2 *>(gb + p.o_mc + h * 256 + 8 * lane);
                        }
                        bm4 = *reinterpret_cast<const uint4 *>(gb + p.o_bm + h * 512 + 16 * lane);
                        const int nb = KOUT >= 0 ? (KOUT + 1) / 2 : p.nb;
                        const uint32_t *ov = reinterpret_cast<const uint32_t *>(gb + p.o_ov + h * 128 * nb + 4 * nb * lane);
                        if (nb == 3) {
                            const uint32_t w0 = ov[0], w1 = ov[1], w2 = ov[2];
                            st[0] = w0 & 0xFFFFFFu;
                            st[1] = (w0 >> 24) | ((w1 & 0xFFFFu) << 8);
                            st[2] = (w1 >> 16) | ((w2 & 0xFFu) << 16);
                            st[3] = w2 >> 8;
                        } else if (nb == 4) {
                            st[0] = ov[0]; st[1] = ov[1]; st[2] = ov[2]; st[3] = ov[3];
                        } else if (nb == 2) {
                            const uint32_t w0 = ov[0], w1 = ov[1];
                            st[0] = w0 & 0xFFFFu; st[1] = w0 >> 16; st[2] = w1 & 0xFFFFu; st[3] = w1 >> 16;
                        } else {
                            const uint32_t w0 = ov[0];
                            st[0] = w0 & 0xFFu; st[1] = (w0 >> 8) & 0xFFu; st[2] = (w0 >> 16) & 0xFFu; st[3] = w0 >> 24;
                        }
                    }
                    OMMX_TR(trk + 3);
                    const uint32_t bmv[4] = {bm4.x, bm4.y, bm4.z, bm4.w};
                    const uint8_t *kreg = gb;                            // k_base region of the group (1 KB aligned)
                    const uint32_t kl_off = (uint32_t)(h * 32 + lane);     // this lane's code byte (channels 4*lane..+3)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int e = (int)(int8_t)(e4 >> (8 * c));
                        const float inv_s = __uint_as_float((uint32_t)(127 - e) << 23);
                        const uint32_t zw = (c & 2) ? z4.y : z4.x;
                        const float zp = bf16_bits_to_f32((c & 1) ? (zw >> 16) : (zw & 0xFFFFu));
                        const float fs = inv_s * pa_f[c];
                        // zp row: zp / scale in slot units (exact power-of-two scaling of a bf16)
                        *reinterpret_cast<__nv_bfloat16 *>(tile + 32 * DT_STRIDE + pa_col[c]) = __float2bfloat16_rn(zp * fs);
                        if (splice) {
                            float A, Bc;
                            if (p.use_map) {
                                const uint32_t msw = (c & 2) ? ms4.y : ms4.x, mcw = (c & 2) ? mc4.y : mc4.x;
                                const float ms = bf16_bits_to_f32((c & 1) ? (msw >> 16) : (msw & 0xFFFFu));
                                const float mc = bf16_bits_to_f32((c & 1) ? (mcw >> 16) : (mcw & 0xFFFFu));
                                A = __fdividef(fs, ms);
                                Bc = (mc - zp) * fs;
                            } else {
                                A = pa_f[c];                              // (lvl*s + zp - zp)/s = lvl
                                Bc = 0.f;
                            }
                            uint32_t bits = bmv[c];
                            const uint32_t stream = st[c];
                            const float nf = -pa_f[c];
                            // delta between the outlier value and the base code it replaces, in code units:
                            // ((lvl/ms + mc) - (code*s + zp)) / s, rounded to bf16 as the reference rounds
                            // its delta (the scaling by 1/s and 4^pc is exact)
                            if (KOUT > 0) {
                                if (__popc(bits) == KOUT) {
#pragma unroll
                                    for (int r = KOUT - 1; r >= 0; --r) {
                                        const int pz = 31 - __clz(bits);
                                        bits ^= 1u << pz;
                                        const uint32_t nib = (stream >> (4 * r)) & 0xFu;
                                        const float cf = (float)((kreg[swz128(kl_off + pz * TS, p.swz)] >> (2 * c)) & 3u);
                                        const float X = fmaf(cf, nf, fmaf(s_lut[nib], A, Bc));
                                        *reinterpret_cast<__nv_bfloat16 *>(tile + pz * DT_STRIDE + pa_col[c]) = __float2bfloat16_rn(X);
                                    }
                                } else {
                                    or_status(p.status, OMMX_ST_BAD_GROUP);   // bitmask and value stream disagree
                                }
                            } else {
                                int r = __popc(bits) - 1;
                                while (bits) {
                                    const int pz = 31 - __clz(bits);
                                    bits ^= 1u << pz;
                                    const uint32_t nib = (r < 8) ? ((stream >> (4 * r)) & 0xFu) : 0u;
                                    --r;
                                    const float cf = (float)((kreg[swz128(kl_off + pz * TS, p.swz)] >> (2 * c)) & 3u);
                                    const float X = fmaf(cf, nf, fmaf(s_lut[nib], A, Bc));
                                    *reinterpret_cast<__nv_bfloat16 *>(tile + pz * DT_STRIDE + pa_col[c]) = __float2bfloat16_rn(X);
                                }
                            }
                        }
                    }
                    __syncwarp();
                }
                OMMX_TR(trk + 4);

                if (lane == 0) mbar_arrive(bar_tfull + 8 * unit);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        }
        __syncthreads();
        __syncthreads();
        return;
    }

    // =========================== MMA warps (phase B) ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 " OMMX_REGS_MMA ";");
    const int unit = warp;
    const int h = unit % H, gsel = unit / H;
    const uint8_t *tile = s_tiles + unit * DT_BYTES;
    const uint32_t tile_s = smem_u32(tile);
    // ---- per-thread constants ----
    // MMA row g carries query head (g % 4) when VFOLD (rows 4..7 repeat rows 0..3), else head g.
    const int row_head = VFOLD ? (g & 3) : g;
    const bool row_ok = row_head < p.gqa;
    // q_static: bf16(q*sm_scale) * 2^-1 * 4^-pc for this lane's head row and 32 channel slots
    uint32_t QS[16];
    {
        const __nv_bfloat16 *qrow = p.q + (int64_t)b * p.q_sb + (int64_t)(h * p.gqa + (row_ok ? row_head : 0)) * p.q_sh;
        // this lane's 32 channels are contiguous: four 16-byte loads when the row allows it
        uint32_t qw[16];
        if ((reinterpret_cast<uintptr_t>(qrow) & 15u) == 0) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 t = reinterpret_cast<const uint4 *>(qrow + 32 * j)[v];
                qw[4 * v] = t.x; qw[4 * v + 1] = t.y; qw[4 * v + 2] = t.z; qw[4 * v + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int v = 0; v < 16; ++v) {
                const uint16_t *q16 = reinterpret_cast<const uint16_t *>(qrow + 32 * j);
                qw[v] = (uint32_t)q16[2 * v] | ((uint32_t)q16[2 * v + 1] << 16);
            }
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int wi = r >> 3, i = r & 7;
            const int e0 = 16 * wi + i, e1 = e0 + 8;                  // channel 32j + e0 / + e1
            const float f = 0.5f / (float)(1 << (2 * pos_class(i)));
            float lo = 0.f, hi = 0.f;
            if (row_ok) {
                lo = bf16_round_f32(bf16_bits_to_f32((qw[e0 >> 1] >> (16 * (e0 & 1))) & 0xFFFFu) * p.sm_scale) * f;
                hi = bf16_round_f32(bf16_bits_to_f32((qw[e1 >> 1] >> (16 * (e1 & 1))) & 0xFFFFu) * p.sm_scale) * f;
            }
            QS[r] = pack_bf16x2(lo, hi);
        }
    }
    // V-fold constants: byte selectors of this row pair's two V scale groups
    const int cgA = g >> 2, cgB = 2 + (g >> 2);
    const uint32_t selA = (uint32_t)(cgA | (cgA << 4) | ((4 + cgA) << 8) | ((4 + cgA) << 12));
    const uint32_t selB = (uint32_t)(cgB | (cgB << 4) | ((4 + cgB) << 8) | ((4 + cgB) << 12));
    // ---- online softmax state (row g of the MMA tile) ----
    float m_run = -INFINITY, l_run = 0.f;
    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float acc_rs[4] = {0.f, 0.f, 0.f, 0.f};      // VFOLD: sum_t P'[row][t]        (x128 offset)
    float acc_vz[4] = {0.f, 0.f, 0.f, 0.f};      // VFOLD: sum_t P[row][t] * vz[t][cg = column]
    uint32_t consumed = 0;

    OMMX_TR(252);
    for (int it = 0; it < n_iters; ++it) {
        const int s = it % NSTAGES;
        const uint32_t ph = (it / NSTAGES) & 1;
        OMMX_TR(8 * it);
        if (!mbar_wait(bar_full + 8 * s, ph)) {
            if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
            m_run = -INFINITY; l_run = 0.f;
            break;
        }
        OMMX_TR(8 * it + 1);
        const int lg = it * GS + gsel;                               // local group of this warp
        if (lg < ngroups && !(p.abl & ABL_NO_COMPUTE)) {
            uint8_t *gb = s_stage + (size_t)s * p.stage_bytes + (size_t)gsel * p.gb_bytes;
            const uint8_t *vreg = gb + p.o_vm;                      // v_main region of the group (1 KB aligned)
            const uint8_t *vsc = gb + p.o_vs + h * 4;                // + token*H*4
            const uint8_t *vzp = gb + p.o_vz + h * 8;                // + token*H*8
            const uint8_t *ksc = gb + p.o_ks + h * 128;

            // ======================= phase B: QK^T =======================
            uint32_t QQ[16];
            {
                const uint4 ea = *reinterpret_cast<const uint4 *>(ksc + 32 * j);
                const uint4 eb = *reinterpret_cast<const uint4 *>(ksc + 32 * j + 16);
                const uint32_t E[8] = {ea.x, ea.y, ea.z, ea.w, eb.x, eb.y, eb.z, eb.w};
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const int wi = r >> 3, i = r & 7, bsel = i & 3;
                    const uint32_t sel = (uint32_t)(bsel | (bsel << 4) | ((4 + bsel) << 8) | ((4 + bsel) << 12));
                    const uint32_t t = __byte_perm(E[4 * wi + (i >> 2)], E[4 * wi + 2 + (i >> 2)], sel);
                    const uint32_t f = lop3_and_xor(t, 0x00FF00FFu, 0x00800080u) << 7;   // 2^(e+1) pair
                    QQ[r] = hmul2_bf16(QS[r], f);
                }
            }
            float C[5][4];
#pragma unroll
            for (int nt = 0; nt < 5; ++nt) { C[nt][0] = C[nt][1] = C[nt][2] = C[nt][3] = 0.f; }
            if (!(p.abl & ABL_NO_K)) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const uint2 kw = *reinterpret_cast<const uint2 *>(gb + swz128((uint32_t)((8 * nt + g) * TS + h * 32 + 8 * j), p.swz));
                    uint32_t R[8];
                    codes_to_bf16x2(kw.x, R);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) mma_bf16(C[nt], QQ[2 * kk], 0u, QQ[2 * kk + 1], 0u, R[2 * kk], R[2 * kk + 1]);
                    codes_to_bf16x2(kw.y, R);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) mma_bf16(C[nt], QQ[8 + 2 * kk], 0u, QQ[8 + 2 * kk + 1], 0u, R[2 * kk], R[2 * kk + 1]);
                }
            }
            OMMX_TR(8 * it + 2);
            // outlier tile (+ zp / -128 rows as n-tile 4), built by the decode warp of this unit
            if (!mbar_wait(bar_tfull + 8 * unit, consumed & 1u)) {
                if (lane == 0) { or_status(p.status, OMMX_ST_TIMEOUT); atomicExch(s_abort, 1); }
                m_run = -INFINITY; l_run = 0.f;
                break;
            }
            OMMX_TR(8 * it + 3);
            {
                const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
                for (int nt = 0; nt < 5; ++nt) {
                    if (nt < 4 && (k_out == 0 || no_outlier)) continue;
                    int row = 8 * nt + rr;
                    if (row >= DT_ROWS) row -= DT_ROWS;              // rows 34..39 alias rows 0..5 (columns unused)
                    const uint32_t base = tile_s + row * DT_STRIDE + 2 * (16 * (mi >> 1) + 8 * (mi & 1));
#pragma unroll
                    for (int kp = 0; kp < 4; ++kp) {
                        uint32_t d0, d1, d2, d3;
                        ldsm_x4(base + 64 * kp, d0, d1, d2, d3);
                        mma_bf16(C[nt], QQ[4 * kp], 0u, QQ[4 * kp + 1], 0u, d0, d1);
                        mma_bf16(C[nt], QQ[4 * kp + 2], 0u, QQ[4 * kp + 3], 0u, d2, d3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * (NSTAGES * unit + (consumed % NSTAGES)));   // the next tile may be built
            ++consumed;
            OMMX_TR(8 * it + 4);
            // q.zp - 128*sum(q'') sits in columns 0 and 1 of n-tile 4 (lanes with j == 0)
            float qzo = C[4][0] + C[4][1];
            qzo = __shfl_sync(0xFFFFFFFFu, qzo, lane & ~3);

            // ======================= online softmax =======================
            float x[8];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) { x[2 * nt] = C[nt][0] + qzo; x[2 * nt + 1] = C[nt][1] + qzo; }
            if (p.logit_cap > 0.f) {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = p.logit_cap * tanhf(x[i] / p.logit_cap);
            }
            const int tok_base = 32 * lg;
            if (tok_base + 32 > ntok) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    if (tok_base + 8 * nt + 2 * j >= ntok) x[2 * nt] = -INFINITY;
                    if (tok_base + 8 * nt + 2 * j + 1 >= ntok) x[2 * nt + 1] = -INFINITY;
                }
            }
            float mloc = x[0];
#pragma unroll
            for (int i = 1; i < 8; ++i) mloc = fmaxf(mloc, x[i]);
            mloc = fmaxf(mloc, __shfl_xor_sync(0xFFFFFFFFu, mloc, 1));
            mloc = fmaxf(mloc, __shfl_xor_sync(0xFFFFFFFFu, mloc, 2));
            const float m_new = fmaxf(m_run, mloc);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = fast_exp2((m_run - m_use) * LOG2E);   // m_run = -inf -> 0
            const float mneg = -m_use * LOG2E;
            float psum = 0.f;
            uint32_t P[4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float p0 = fast_exp2(fmaf(x[2 * nt], LOG2E, mneg));
                const float p1 = fast_exp2(fmaf(x[2 * nt + 1], LOG2E, mneg));
                psum += p0 + p1;
                P[nt] = pack_bf16x2(p0, p1);
            }
            l_run = l_run * corr + psum;
            m_run = m_new;
            if (__any_sync(0xFFFFFFFFu, corr != 1.0f)) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    acc[i][0] *= corr; acc[i][1] *= corr;
                    if (VFOLD) { acc[i][2] *= corr; acc[i][3] *= corr; }
                }
                if (VFOLD) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) { acc_rs[i] *= corr; acc_vz[i] *= corr; }
                }
            }

            OMMX_TR(8 * it + 5);
            // ======================= P.V =======================
            // lane (g, j) supplies channel column g of every n-tile: channels 16*g + i, scale group g/2
            if (!(p.abl & ABL_NO_V)) {
                if (VFOLD) {
                    // P'[row][t] = P[head][t] * 2^(e_v[t][cg(row)] + 1)   (exact)
                    uint32_t PA[4], PB[4];
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const int ta = 8 * nt + 2 * j;
                        const uint32_t wa = *reinterpret_cast<const uint32_t *>(vsc + ta * H * 4);
                        const uint32_t wb = *reinterpret_cast<const uint32_t *>(vsc + (ta + 1) * H * 4);
                        const uint32_t fa = lop3_and_xor(__byte_perm(wa, wb, selA), 0x00FF00FFu, 0x00800080u) << 7;
                        const uint32_t fb = lop3_and_xor(__byte_perm(wa, wb, selB), 0x00FF00FFu, 0x00800080u) << 7;
                        PA[nt] = hmul2_bf16(P[nt], fa);
                        PB[nt] = hmul2_bf16(P[nt], fb);
                    }
#pragma unroll
                    for (int kt = 0; kt < 2; ++kt) {
                        const int ta = 16 * kt + 2 * j;
                        const uint32_t wa = *reinterpret_cast<const uint32_t *>(vreg + swz128((uint32_t)(ta * TS + h * 32 + 4 * g), p.swz));
                        const uint32_t wb = *reinterpret_cast<const uint32_t *>(vreg + swz128((uint32_t)((ta + 1) * TS + h * 32 + 4 * g), p.swz));
                        const uint32_t wc = *reinterpret_cast<const uint32_t *>(vreg + swz128((uint32_t)((ta + 8) * TS + h * 32 + 4 * g), p.swz));
                        const uint32_t wd = *reinterpret_cast<const uint32_t *>(vreg + swz128((uint32_t)((ta + 9) * TS + h * 32 + 4 * g), p.swz));
                        uint32_t R0[8], R1[8];
                        codes_to_bf16x2(__byte_perm(wa, wb, 0x5410), R0);       // channels 0..7 of (ta, tb)
                        codes_to_bf16x2(__byte_perm(wc, wd, 0x5410), R1);
#pragma unroll
                        for (int i = 0; i < 8; ++i) mma_bf16(acc[i], PA[2 * kt], PB[2 * kt], PA[2 * kt + 1], PB[2 * kt + 1], R0[i], R1[i]);
                        codes_to_bf16x2(__byte_perm(wa, wb, 0x7632), R0);       // channels 8..15
                        codes_to_bf16x2(__byte_perm(wc, wd, 0x7632), R1);
#pragma unroll
                        for (int i = 0; i < 8; ++i) mma_bf16(acc[8 + i], PA[2 * kt], PB[2 * kt], PA[2 * kt + 1], PB[2 * kt + 1], R0[i], R1[i]);
                        // row sums of P' (the magic +128 of every raw V value comes back out through them)
                        mma_bf16(acc_rs, PA[2 * kt], PB[2 * kt], PA[2 * kt + 1], PB[2 * kt + 1], 0x3F803F80u, 0x3F803F80u);
                        // zero-point bias: column n = scale group n (n < 4), B[k = token][n] = vz[token][n]
                        uint32_t z0 = 0u, z1 = 0u;
                        if (g < 4) {
                            z0 = (uint32_t)*reinterpret_cast<const uint16_t *>(vzp + ta * H * 8 + 2 * g)
                               | ((uint32_t)*reinterpret_cast<const uint16_t *>(vzp + (ta + 1) * H * 8 + 2 * g) << 16);
                            z1 = (uint32_t)*reinterpret_cast<const uint16_t *>(vzp + (ta + 8) * H * 8 + 2 * g)
                               | ((uint32_t)*reinterpret_cast<const uint16_t *>(vzp + (ta + 9) * H * 8 + 2 * g) << 16);
                        }
                        mma_bf16(acc_vz, P[2 * kt], P[2 * kt], P[2 * kt + 1], P[2 * kt + 1], z0, z1);
                    }
                } else {
#pragma unroll
                    for (int kt = 0; kt < 2; ++kt) {
                        uint32_t Vr[2][16];
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int ta = 16 * kt + 8 * half + 2 * j, tb = ta + 1;
                            const uint32_t wa = *reinterpret_cast<const uint32_t *>(vreg + swz128((uint32_t)(ta * TS + h * 32 + 4 * g), p.swz));
                            const uint32_t wb = *reinterpret_cast<const uint32_t *>(vreg + swz128((uint32_t)(tb * TS + h * 32 + 4 * g), p.swz));
                            const uint32_t ea = vsc[ta * H * 4 + (g >> 1)], eb2 = vsc[tb * H * 4 + (g >> 1)];
                            const uint32_t za = *reinterpret_cast<const uint16_t *>(vzp + ta * H * 8 + 2 * (g >> 1));
                            const uint32_t zb = *reinterpret_cast<const uint16_t *>(vzp + tb * H * 8 + 2 * (g >> 1));
                            const uint32_t vs2 = (((ea | (eb2 << 16)) ^ 0x00800080u) & 0x00FF00FFu) << 7;   // 2^(e+1) pair
                            const uint32_t vz2 = za | (zb << 16);
                            const uint32_t vs_p0 = hmul2_bf16(vs2, 0x3F003F00u);    // * 2^-1
                            const uint32_t vs_p1 = hmul2_bf16(vs2, 0x3E003E00u);    // * 2^-3
                            const uint32_t vs_p2 = hmul2_bf16(vs2, 0x3D003D00u);    // * 2^-5
                            uint32_t R[8];
                            const uint32_t K128 = 0x43004300u;
                            codes_to_bf16x2(__byte_perm(wa, wb, 0x5410), R);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int pc = pos_class(i);
                                Vr[half][i] = hfma2_bf16(hsub2_bf16(R[i], K128), pc == 0 ? vs_p0 : (pc == 1 ? vs_p1 : vs_p2), vz2);
                            }
                            codes_to_bf16x2(__byte_perm(wa, wb, 0x7632), R);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int pc = pos_class(i);
                                Vr[half][8 + i] = hfma2_bf16(hsub2_bf16(R[i], K128), pc == 0 ? vs_p0 : (pc == 1 ? vs_p1 : vs_p2), vz2);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i) mma_bf16(acc[i], P[2 * kt], 0u, P[2 * kt + 1], 0u, Vr[0][i], Vr[1][i]);
                    }
                }
            }
        }
        // release the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        OMMX_TR(8 * it + 6);
    }
    OMMX_TR(253);

    // ---- epilogue: finalize this lane's 32 output channels, merge warps that share a head ----
    // Every lane ends up with outv[0..15] = channels 32j + i and outv[16..31] = channels 32j + 16 + i of
    // one (head, split) row, un-normalised; `useful` marks the lanes whose row is real.
    float l_tot = l_run;
    l_tot += __shfl_xor_sync(0xFFFFFFFFu, l_tot, 1);
    l_tot += __shfl_xor_sync(0xFFFFFFFFu, l_tot, 2);
    float outv[32];
    bool useful;
    if (VFOLD) {
        // lane (g, j): columns 2j, 2j+1 are channels of scale group j; row g has group g/4, row g+8 group 2+g/4
        const bool lo_row = (g >> 2) == j, hi_row = (2 + (g >> 2)) == j;
        useful = row_ok && (lo_row || hi_row);
        const float rs = hi_row ? acc_rs[2] : acc_rs[0];
        // bias of (head, group j) sits in lane (g, j/2), register j&1
        const float b0 = __shfl_sync(0xFFFFFFFFu, acc_vz[0], (lane & ~3) | (j >> 1));
        const float b1 = __shfl_sync(0xFFFFFFFFu, acc_vz[1], (lane & ~3) | (j >> 1));
        const float bias = (j & 1) ? b1 : b0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float f = 0.5f / (float)(1 << (2 * pos_class(i & 7)));
            const float a0 = hi_row ? acc[i][2] : acc[i][0], a1 = hi_row ? acc[i][3] : acc[i][1];
            outv[i] = fmaf(a0 - 128.f * rs, f, bias);
            outv[16 + i] = fmaf(a1 - 128.f * rs, f, bias);
        }
    } else {
        useful = row_ok;
#pragma unroll
        for (int i = 0; i < 16; ++i) { outv[i] = acc[i][0]; outv[16 + i] = acc[i][1]; }
    }
    const int out_head = h * p.gqa + row_head;

    // Wait for every warp (and the producer) before the ring memory is reused as scratch.
    __syncthreads();
    float *scratch = reinterpret_cast<float *>(s_stage);             // [NCW][32 lanes][34]
    if (GS > 1 && gsel > 0) {
        float *my = scratch + ((size_t)unit * 32 + lane) * 34;
        my[0] = m_run; my[1] = l_tot;
#pragma unroll
        for (int i = 0; i < 32; ++i) my[2 + i] = outv[i];
    }
    __syncthreads();
    if (gsel == 0) {
        for (int o = 1; o < GS; ++o) {
            const float *ot = scratch + ((size_t)(o * H + h) * 32 + lane) * 34;
            const float m2 = ot[0], l2 = ot[1];
            const float mn = fmaxf(m_run, m2);
            const float mu = (mn == -INFINITY) ? 0.f : mn;
            const float c1 = fast_exp2((m_run - mu) * LOG2E), c2 = fast_exp2((m2 - mu) * LOG2E);
            l_tot = l_tot * c1 + l2 * c2;
#pragma unroll
            for (int i = 0; i < 32; ++i) outv[i] = outv[i] * c1 + ot[2 + i] * c2;
            m_run = mn;
        }
        if (useful) {
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            float *dst = p.al + (int64_t)b * p.al_sb + (int64_t)out_head * p.al_sh + (int64_t)split * p.al_ss;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                dst[32 * j + i] = outv[i] * inv;
                dst[32 * j + 16 + i] = outv[16 + i] * inv;
            }
            const bool lse_writer = VFOLD ? (g < 4 && j == 0) : (j == 0);
            if (lse_writer) dst[HD] = l_tot > 0.f ? m_run + logf(l_tot) : -INFINITY;
        }
    }
    OMMX_TR(254);
}

// =================================================================================================
// Stage 2: bf16 sink/recent rows + log-sum-exp combine (reference: paged_decode.py:2366-2500)
// =================================================================================================
struct S2Params {
    const __nv_bfloat16 *q;
    int64_t q_sb, q_sh;
    int32_t Hq, gqa, D;
    const __nv_bfloat16 *k_tail, *v_tail;
    int64_t t_sb, t_st, t_sh;
    const int32_t *b_tail_len, *b_seq_len;
    int32_t max_tail;
    const float *al;
    int64_t al_sb, al_sh, al_ss;
    int32_t S;
    void *o;
    int32_t o_bf16;
    int64_t o_sb, o_sh;
    float *lse;
    int64_t lse_sb;
    float sm_scale, logit_cap;
};

constexpr int S2_THREADS = 512;
constexpr int S2_WARPS = S2_THREADS / 32;
constexpr int S2_MAX_TAIL = 256;
constexpr int S2_MAX_SPLITS = 1024;

// One CTA per (query head, sequence).  Warps stripe over the bf16 residual rows for the logits,
// then over the splits for the combine; every loop keeps many independent loads in flight,
// because this kernel is pure latency (a few hundred KB through L2).
__global__ void __launch_bounds__(S2_THREADS) decode_stage2_kernel(const S2Params p) {
    __shared__ float s_q[HD];
    __shared__ float s_logit[S2_MAX_TAIL];
    __shared__ float s_w[S2_MAX_SPLITS];
    __shared__ float s_red[S2_WARPS];
    __shared__ float s_acc[S2_WARPS][HD];
    const int hq = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = hq / p.gqa;
    const int seq = p.b_seq_len[b];
    int tail = p.b_tail_len ? p.b_tail_len[b] : 0;
    tail = max(0, min(tail, min(p.max_tail, S2_MAX_TAIL)));
    const int D = p.D;                                                   // == HD
    const int per = (seq > 0 && p.S > 0) ? (((seq + p.S - 1) / p.S) + 31) / 32 * 32 : 0;
    const int nsplit = per > 0 ? min(p.S, (seq + per - 1) / per) : 0;    // splits s with s*per < seq
    const float *base = p.al + (int64_t)b * p.al_sb + (int64_t)hq * p.al_sh;

    // ---- bf16 residual rows: logits of this q head (independent of stage 1) ----
    if (tail > 0) {
        if (tid < D) s_q[tid] = __bfloat162float(p.q[(int64_t)b * p.q_sb + (int64_t)hq * p.q_sh + tid]);
        __syncthreads();
        const __nv_bfloat16 *kt = p.k_tail + (int64_t)b * p.t_sb + (int64_t)kvh * p.t_sh;
        for (int r = warp; r < tail; r += S2_WARPS) {
            const uint2 kv = *reinterpret_cast<const uint2 *>(kt + (int64_t)r * p.t_st + 4 * lane);
            float d = s_q[4 * lane] * bf16_bits_to_f32(kv.x & 0xFFFFu) + s_q[4 * lane + 1] * bf16_bits_to_f32(kv.x >> 16)
                    + s_q[4 * lane + 2] * bf16_bits_to_f32(kv.y & 0xFFFFu) + s_q[4 * lane + 3] * bf16_bits_to_f32(kv.y >> 16);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
            if (lane == 0) {
                float x = d * p.sm_scale;
                if (p.logit_cap > 0.f) x = p.logit_cap * tanhf(x / p.logit_cap);
                s_logit[r] = x;
            }
        }
    }
    // ---- everything below reads what stage 1 wrote: wait for that grid (no-op without a
    //      programmatic launch) ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float mloc = -INFINITY;
    for (int s = tid; s < nsplit; s += S2_THREADS) {
        const float l = base[(int64_t)s * p.al_ss + D];
        s_w[s] = l;
        mloc = fmaxf(mloc, l);
    }
    __syncthreads();
    // ---- global max over split lse values and residual logits ----
    for (int r = tid; r < tail; r += S2_THREADS) mloc = fmaxf(mloc, s_logit[r]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xFFFFFFFFu, mloc, o));
    if (lane == 0) s_red[warp] = mloc;
    __syncthreads();
    float g_max = s_red[0];
#pragma unroll
    for (int w = 1; w < S2_WARPS; ++w) g_max = fmaxf(g_max, s_red[w]);
    const float g_safe = (g_max == -INFINITY) ? 0.f : g_max;
    __syncthreads();
    // weights: splits enter with exp(lse_s - max), residual rows with exp(logit - max)
    float wsum = 0.f;
    for (int s = tid; s < nsplit; s += S2_THREADS) { const float w = __expf(s_w[s] - g_safe); s_w[s] = w; wsum += w; }
    for (int r = tid; r < tail; r += S2_THREADS) { const float w = __expf(s_logit[r] - g_safe); s_logit[r] = w; wsum += w; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xFFFFFFFFu, wsum, o);
    if (lane == 0) s_red[warp] = wsum;
    __syncthreads();
    float den = 0.f;
#pragma unroll
    for (int w = 0; w < S2_WARPS; ++w) den += s_red[w];

    // ---- weighted sum: warp w takes splits / rows w, w+16, ...; lane owns channels lane + 32*i ----
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
    for (int s = warp; s < nsplit; s += S2_WARPS) {
        const float *row = base + (int64_t)s * p.al_ss;
        const float w = s_w[s];
        a0 += w * row[lane]; a1 += w * row[lane + 32]; a2 += w * row[lane + 64]; a3 += w * row[lane + 96];
    }
    if (tail > 0) {
        const __nv_bfloat16 *vt = p.v_tail + (int64_t)b * p.t_sb + (int64_t)kvh * p.t_sh;
#pragma unroll 4
        for (int r = warp; r < tail; r += S2_WARPS) {
            const __nv_bfloat16 *row = vt + (int64_t)r * p.t_st;
            const float w = s_logit[r];
            a0 += w * __bfloat162float(row[lane]); a1 += w * __bfloat162float(row[lane + 32]);
            a2 += w * __bfloat162float(row[lane + 64]); a3 += w * __bfloat162float(row[lane + 96]);
        }
    }
    s_acc[warp][lane] = a0; s_acc[warp][lane + 32] = a1;
    s_acc[warp][lane + 64] = a2; s_acc[warp][lane + 96] = a3;
    __syncthreads();
    if (tid < D) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < S2_WARPS; ++w) acc += s_acc[w][tid];
        const float out = acc / (den > 0.f ? den : 1.f);
        if (p.o_bf16) reinterpret_cast<__nv_bfloat16 *>(p.o)[(int64_t)b * p.o_sb + (int64_t)hq * p.o_sh + tid] = __float2bfloat16_rn(out);
        else reinterpret_cast<float *>(p.o)[(int64_t)b * p.o_sb + (int64_t)hq * p.o_sh + tid] = out;
        if (tid == 0) p.lse[(int64_t)b * p.lse_sb + hq] = g_max + logf(den);
    }
}

// =================================================================================================
// merge of partial softmax states (reference: paged_decode.py:2650-2690)
// =================================================================================================
__global__ void __launch_bounds__(128) merge_states_kernel(const float *o_parts, const float *lse_parts,
                                                           const int32_t *valid, int P, int R, int D,
                                                           float *o, float *lse) {
    const int r = blockIdx.x;
    int np = P;
    if (valid) { int v = valid[r]; if (v >= 0) np = min(v, P); }
    float m = -INFINITY;
    for (int q = 0; q < np; ++q) m = fmaxf(m, lse_parts[(int64_t)q * R + r]);
    const float ms = (m == -INFINITY) ? 0.f : m;
    float den = 0.f;
    for (int q = 0; q < np; ++q) den += __expf(lse_parts[(int64_t)q * R + r] - ms);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int q = 0; q < np; ++q)
            acc += __expf(lse_parts[(int64_t)q * R + r] - ms) * o_parts[((int64_t)q * R + r) * D + d];
        o[(int64_t)r * D + d] = acc / (den > 0.f ? den : 1.f);
    }
    if (threadIdx.x == 0) lse[r] = ms + logf(den);
}

// =================================================================================================
// host side
// =================================================================================================
static int validate_decode(const ommx_decode_args *a) {
    if (!a) return fail(OMMX_E_ARG, "decode: null args");
    const ommx_kv_planes &pl = a->planes;
    if (!a->q || !a->o || !a->lse || !a->attn_logits || !a->b_seq_len)
        return fail(OMMX_E_ARG, "decode: q/o/lse/attn_logits/b_seq_len must not be null");
    if (a->q_dtype != OMMX_DT_BF16) return fail(OMMX_E_UNSUPPORTED, "decode: q must be bf16");
    if (a->o_dtype != OMMX_DT_F32 && a->o_dtype != OMMX_DT_BF16) return fail(OMMX_E_UNSUPPORTED, "decode: o must be f32 or bf16");
    if (pl.head_dim != HD) return fail(OMMX_E_UNSUPPORTED, "decode: head_dim=%d (this build serves %d)", pl.head_dim, HD);
    if (pl.n_kv_heads != 1 && pl.n_kv_heads != 2 && pl.n_kv_heads != 4 && pl.n_kv_heads != 8)
        return fail(OMMX_E_UNSUPPORTED, "decode: n_kv_heads=%d per device must be 1, 2, 4 or 8", pl.n_kv_heads);
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_q_heads % pl.n_kv_heads != 0)
        return fail(OMMX_E_ARG, "decode: batch=%d n_q_heads=%d n_kv_heads=%d", a->batch, a->n_q_heads, pl.n_kv_heads);
    if (a->n_q_heads / pl.n_kv_heads > 8)
        return fail(OMMX_E_UNSUPPORTED, "decode: GQA group of %d query heads per kv head (max 8)", a->n_q_heads / pl.n_kv_heads);
    if (pl.page_size != 8 && pl.page_size != 16 && pl.page_size != 32)
        return fail(OMMX_E_UNSUPPORTED, "decode: page_size=%d must be 8, 16 or 32", pl.page_size);
    if (pl.scale_kind != OMMX_SCALE_INT8_EXP)
        return fail(OMMX_E_UNSUPPORTED, "decode: only int8 power-of-two scale planes are served (pack with use_pow2)");
    if (pl.outliers_per_vector < 0 || pl.outliers_per_vector > 8)
        return fail(OMMX_E_UNSUPPORTED, "decode: outliers_per_vector=%d outside [0,8]", pl.outliers_per_vector);
    if (a->packed_start_offset != 0) return fail(OMMX_E_UNSUPPORTED, "decode: packed_start_offset must be 0");
    if (a->seg_group_base < 0) return fail(OMMX_E_ARG, "decode: seg_group_base=%d", a->seg_group_base);
    if (a->num_kv_splits < 1) return fail(OMMX_E_ARG, "decode: num_kv_splits=%d", a->num_kv_splits);
    if (a->num_kv_splits > S2_MAX_SPLITS) return fail(OMMX_E_UNSUPPORTED, "decode: num_kv_splits=%d (max %d)", a->num_kv_splits, S2_MAX_SPLITS);
    if (a->max_tail_len > S2_MAX_TAIL) return fail(OMMX_E_UNSUPPORTED, "decode: max_tail_len=%d (max %d)", a->max_tail_len, S2_MAX_TAIL);
    if (a->max_tail_len > 0 && (!a->k_tail || !a->v_tail || !a->b_tail_len))
        return fail(OMMX_E_ARG, "decode: max_tail_len>0 needs k_tail, v_tail and b_tail_len");
    if (a->max_seq_len > 0) {
        if (!a->req_to_token || !a->req_to_group) return fail(OMMX_E_ARG, "decode: page / group tables are null");
        if (!pl.k_base || !pl.k_scale || !pl.k_zp || !pl.v_main || !pl.v_scale || !pl.v_zp)
            return fail(OMMX_E_ARG, "decode: a KV plane is null");
        if (pl.outliers_per_vector > 0 && (!pl.k_obmp || !pl.k_oval))
            return fail(OMMX_E_ARG, "decode: k>0 needs k_obmp and k_oval");
        if (pl.outliers_per_vector > 0 && pl.kv_outlier_map && (!pl.k_mapscale || !pl.k_mapcenter))
            return fail(OMMX_E_ARG, "decode: kv_outlier_map needs k_mapscale and k_mapcenter");
        const void *pp[] = {pl.k_base, pl.k_scale, pl.k_zp, pl.k_obmp, pl.k_oval, pl.k_mapscale, pl.k_mapcenter,
                            pl.v_main, pl.v_scale, pl.v_zp};
        for (const void *x : pp)
            if (((uintptr_t)x & 15) != 0) return fail(OMMX_E_ARG, "decode: every KV plane must be 16-byte aligned");
        const int min_s = ommx_b200_min_num_kv_splits(a->max_seq_len, pl.page_size);
        if (a->num_kv_splits < min_s)
            return fail(OMMX_E_ARG, "decode: num_kv_splits=%d too small for max_seq_len=%d (need >= %d)",
                        a->num_kv_splits, a->max_seq_len, min_s);
    }
    if (a->al_stride_s < HD + 1) return fail(OMMX_E_ARG, "decode: attn_logits last dim must be head_dim+1");
    return 0;
}

// ---- tensor maps of the code planes (driver entry point looked up at run time, no link dependency) ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static std::atomic<int> state{0};                 // 0 unknown, 1 found, 2 absent
    static EncodeTiledFn fn = nullptr;
    int st = state.load(std::memory_order_acquire);
    if (st == 0) {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        const bool ok = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
                        q == cudaDriverEntryPointSuccess && f != nullptr;
        if (ok) fn = reinterpret_cast<EncodeTiledFn>(f);
        (void)cudaGetLastError();
        state.store(ok ? 1 : 2, std::memory_order_release);
        st = ok ? 1 : 2;
    }
    return st == 1 ? fn : nullptr;
}

// Plane viewed as [bytes/128][128] uint8, box = one page, 128-byte swizzle.  Returns false when the
// map cannot be built (the caller then stages the plane with plain bulk copies).
// Encoded maps are kept in a small table keyed by (base, bytes, box rows): a serving loop calls with the
// same planes every step and the driver call costs about a microsecond.
static bool make_code_map(CUtensorMap *m, const void *base, int64_t total_bytes, int rows_per_page) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || total_bytes < 128 || rows_per_page < 8 || rows_per_page > 256) return false;
    struct Entry { const void *base; int64_t bytes; int rows; CUtensorMap map; };
    constexpr int N = 256;
    static Entry table[N];
    static std::mutex mu;
    const size_t slot = (reinterpret_cast<uintptr_t>(base) >> 8) % N;
    {
        std::lock_guard<std::mutex> g(mu);
        const Entry &e = table[slot];
        if (e.base == base && e.bytes == total_bytes && e.rows == rows_per_page) { *m = e.map; return true; }
    }
    cuuint64_t gdim[2] = {128, (cuuint64_t)(total_bytes / 128)};
    cuuint64_t gstride[1] = {128};
    cuuint32_t box[2] = {128, (cuuint32_t)rows_per_page};
    cuuint32_t estr[2] = {1, 1};
    if (fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), gdim, gstride, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> g(mu);
    table[slot].base = base; table[slot].bytes = total_bytes; table[slot].rows = rows_per_page; table[slot].map = *m;
    return true;
}

static size_t stage1_smem(const S1Params &p) {
    return 1024 + (size_t)NSTAGES * p.stage_bytes + (size_t)NCW * DT_BYTES + (MAX_SPLIT_GROUPS + MAX_SPLIT_PAGES) * 4 + 64
           + (2 * NSTAGES + (1 + NSTAGES) * NCW) * 8 + 16 + MAX_STAGE_COPIES * sizeof(CopyDesc);
}

template <int KOUT, bool VFOLD>
static int launch_s1(const S1Params &p, dim3 grid, size_t smem, cudaStream_t st) {
    static size_t attr_smem = 0;                       // one per instantiation
    if (smem > attr_smem) {
        OMMX_CUDA_TRY(cudaFuncSetAttribute(decode_stage1_kernel<KOUT, VFOLD>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem = smem;
    }
    decode_stage1_kernel<KOUT, VFOLD><<<grid, S1_THREADS, smem, st>>>(p);
    OMMX_CUDA_TRY(cudaGetLastError());
    count_launch();
    return 0;
}

static int launch_stage1(const ommx_decode_args *a, cudaStream_t st) {
    if (a->max_seq_len <= 0) return 0;                                   // tail-only decode
    const ommx_kv_planes &pl = a->planes;
    S1Params p;
    p.q = (const __nv_bfloat16 *)a->q; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h;
    p.B = a->batch; p.Hq = a->n_q_heads; p.H = pl.n_kv_heads; p.gqa = a->n_q_heads / pl.n_kv_heads;
    p.k_base = (const uint8_t *)pl.k_base; p.v_main = (const uint8_t *)pl.v_main;
    p.v_scale = (const uint8_t *)pl.v_scale; p.v_zp = (const uint8_t *)pl.v_zp;
    p.k_scale = (const uint8_t *)pl.k_scale; p.k_zp = (const uint8_t *)pl.k_zp;
    p.k_ms = (const uint8_t *)pl.k_mapscale; p.k_mc = (const uint8_t *)pl.k_mapcenter;
    p.k_obmp = (const uint8_t *)pl.k_obmp; p.k_oval = (const uint8_t *)pl.k_oval;
    p.ps = pl.page_size; p.ppg = 32 / pl.page_size; p.num_pages = pl.num_pages; p.num_slots = pl.num_group_slots;
    p.k_out = pl.outliers_per_vector; p.nb = (pl.outliers_per_vector + 1) / 2;
    p.use_map = (pl.kv_outlier_map && pl.outliers_per_vector > 0) ? 1 : 0;
    p.b_seq_len = a->b_seq_len; p.r2t = a->req_to_token; p.r2g = a->req_to_group; p.tbl64 = a->table_is_int64;
    p.r2t_sb = a->r2t_stride_b; p.r2g_sb = a->r2g_stride_b;
    p.al = a->attn_logits; p.al_sb = a->al_stride_b; p.al_sh = a->al_stride_h; p.al_ss = a->al_stride_s;
    p.S = a->num_kv_splits; p.seg_group_base = a->seg_group_base;
    p.sm_scale = a->sm_scale; p.logit_cap = a->logit_cap; p.status = a->status;
    const int H = p.H;
    p.GS = NCW / H;
    p.o_vm = H * 1024; p.o_vs = H * 2048; p.o_vz = p.o_vs + H * 128; p.o_ks = p.o_vz + H * 256;
    p.o_kz = p.o_ks + H * 128; p.o_ms = p.o_kz + H * 256; p.o_mc = p.o_ms + H * 256; p.o_bm = p.o_mc + H * 256;
    p.o_ov = p.o_bm + H * 512;
    p.gb_bytes = p.o_ov + H * 128 * (p.nb > 0 ? p.nb : 0);
    // swizzled tensor-map staging of the two code planes when a page is whole 1 KB swizzle atoms and
    // the 1 KB rounding of the group block still fits shared memory (4 or 8 local kv heads)
    const int64_t page_bytes = (int64_t)p.ps * H * 32;
    p.swz = 0;
    p.rows_per_page = (int32_t)(page_bytes / 128);
    memset(&p.tmap_k, 0, sizeof(CUtensorMap));
    memset(&p.tmap_v, 0, sizeof(CUtensorMap));
    if (H >= 4 && page_bytes % 1024 == 0 &&
        make_code_map(&p.tmap_k, pl.k_base, (int64_t)pl.num_pages * page_bytes, p.rows_per_page) &&
        make_code_map(&p.tmap_v, pl.v_main, (int64_t)pl.num_pages * page_bytes, p.rows_per_page))
        p.swz = 0x70u;
    const int round_to = p.swz ? 1024 : 128;
    p.gb_bytes = (p.gb_bytes + round_to - 1) / round_to * round_to;
    p.stage_bytes = p.GS * p.gb_bytes;
    p.abl = a->abl_flags;
    const size_t smem = stage1_smem(p);
    dim3 grid(a->num_kv_splits, a->batch);
    const bool vfold = p.gqa <= 4;
    if (p.k_out == 6) return vfold ? launch_s1<6, true>(p, grid, smem, st) : launch_s1<6, false>(p, grid, smem, st);
    if (p.k_out == 0) return vfold ? launch_s1<0, true>(p, grid, smem, st) : launch_s1<0, false>(p, grid, smem, st);
    return vfold ? launch_s1<-1, true>(p, grid, smem, st) : launch_s1<-1, false>(p, grid, smem, st);
}

// `after_stage1`: the previous kernel in the stream is this call's own stage 1, so stage 2 may be
// launched as its programmatic dependent.
static int launch_stage2(const ommx_decode_args *a, cudaStream_t st, bool after_stage1 = false) {
    const ommx_kv_planes &pl = a->planes;
    S2Params p;
    p.q = (const __nv_bfloat16 *)a->q; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h;
    p.Hq = a->n_q_heads; p.gqa = a->n_q_heads / pl.n_kv_heads; p.D = pl.head_dim;
    p.k_tail = (const __nv_bfloat16 *)a->k_tail; p.v_tail = (const __nv_bfloat16 *)a->v_tail;
    p.t_sb = a->tail_stride_b; p.t_st = a->tail_stride_t; p.t_sh = a->tail_stride_h;
    p.b_tail_len = a->max_tail_len > 0 ? a->b_tail_len : nullptr; p.b_seq_len = a->b_seq_len;
    p.max_tail = a->max_tail_len;
    p.al = a->attn_logits; p.al_sb = a->al_stride_b; p.al_sh = a->al_stride_h; p.al_ss = a->al_stride_s;
    p.S = a->max_seq_len > 0 ? a->num_kv_splits : 0;
    p.o = a->o; p.o_bf16 = (a->o_dtype == OMMX_DT_BF16); p.o_sb = a->o_stride_b; p.o_sh = a->o_stride_h;
    p.lse = a->lse; p.lse_sb = a->lse_stride_b;
    p.sm_scale = a->sm_scale; p.logit_cap = a->logit_cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a->n_q_heads, a->batch);
    cfg.blockDim = dim3(S2_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;   // overlap this kernel's prologue with stage 1's tail
    cfg.attrs = attr;
    cfg.numAttrs = (after_stage1 && a->max_seq_len > 0) ? 1 : 0;
    OMMX_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_stage2_kernel, p));
    count_launch();
    return 0;
}

}  // namespace ommx

extern "C" int ommx_b200_min_num_kv_splits(int32_t max_seq_len, int32_t page_size) {
    using namespace ommx;
    if (max_seq_len <= 0) return 1;
    int ppg = page_size > 0 && page_size <= 32 ? 32 / page_size : 1;
    int max_groups = MAX_SPLIT_GROUPS;
    if (max_groups * ppg > MAX_SPLIT_PAGES) max_groups = MAX_SPLIT_PAGES / ppg;
    const int groups = (max_seq_len + 31) / 32;
    return (groups + max_groups - 1) / max_groups;
}

extern "C" int ommx_b200_auto_num_kv_splits(int32_t max_seq_len, int32_t batch, int32_t n_kv_heads) {
    (void)n_kv_heads;                       // one CTA serves all local kv heads of its token range
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            sm_count = n;
        else
            sm_count = 148;
    }
    const int groups = max(1, (max_seq_len + 31) / 32);
    const int b = max(1, batch);
    int s = (sm_count + b - 1) / b;                                       // one CTA per SM
    if (b > 1) s = max(s, min(8, groups / 16));                           // ragged batches: finer grain
    s = min(s, groups);
    s = max(s, ommx_b200_min_num_kv_splits(max_seq_len, 16));
    return max(1, s);
}

extern "C" int ommx_b200_decode_stage1(const ommx_decode_args *a, void *stream) {
    int rc = ommx::validate_decode(a);
    if (rc) return rc;
    return ommx::launch_stage1(a, (cudaStream_t)stream);
}
extern "C" int ommx_b200_decode_stage2(const ommx_decode_args *a, void *stream) {
    int rc = ommx::validate_decode(a);
    if (rc) return rc;
    return ommx::launch_stage2(a, (cudaStream_t)stream);
}
extern "C" int ommx_b200_decode(const ommx_decode_args *a, void *stream) {
    int rc = ommx::validate_decode(a);
    if (rc) return rc;
    rc = ommx::launch_stage1(a, (cudaStream_t)stream);
    if (rc) return rc;
    return ommx::launch_stage2(a, (cudaStream_t)stream, true);
}

// -------------------------------------------------------------------------------------------------
// Decode with the split workspace owned by the library.
//
// Some hosts that embed this library may not allocate device memory at all on their serving path:
// a runtime whose allocator has been frozen after start-up (every later cudaMalloc would fragment or
// overrun a pool sized to the last megabyte), or a plug-in that is handed tensors but no allocator.
// ommx_b200_decode needs a workspace for the per-split partial results; this entry point takes it
// from a fixed array inside the library image instead, so the caller passes only inputs and outputs.
// The array is part of the module: every GPU that loads the library holds its 8 MiB until exit.
constexpr size_t STATIC_WS_FLOATS = (size_t)2 << 20;                      // 2 Mi floats = 8 MiB
static __device__ __align__(256) float g_static_ws[STATIC_WS_FLOATS];

// In host code the name g_static_ws is only a handle, not a device address; the address each
// device gave the array is asked for once per device, with that device current, and kept.
static int static_ws_address(float **out) {
    static std::atomic<float *> cache[64];
    int dev = -1;
    OMMX_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ommx::fail(OMMX_E_UNSUPPORTED, "decode_static_ws: device ordinal %d", dev);
    float *ptr = cache[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        void *sym = nullptr;
        OMMX_CUDA_TRY(cudaGetSymbolAddress(&sym, g_static_ws));
        if (sym == nullptr) return ommx::fail(OMMX_E_CUDA, "decode_static_ws: the workspace symbol has no address on device %d", dev);
        ptr = static_cast<float *>(sym);
        cache[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return 0;
}

extern "C" int ommx_b200_decode_static_ws(const ommx_decode_args *a, void *stream) {
    using namespace ommx;
    if (!a) return fail(OMMX_E_ARG, "decode_static_ws: null args");
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->num_kv_splits <= 0)
        return fail(OMMX_E_ARG, "decode_static_ws: batch=%d n_q_heads=%d num_kv_splits=%d", a->batch, a->n_q_heads, a->num_kv_splits);
    const size_t row = (size_t)HD + 1;
    const size_t need = (size_t)a->batch * a->n_q_heads * a->num_kv_splits * row;
    if (need > STATIC_WS_FLOATS)
        return fail(OMMX_E_ARG, "decode_static_ws: batch*n_q_heads*num_kv_splits*(head_dim+1) = %zu floats exceeds the "
                                "built-in workspace of %zu floats (8 MiB); use ommx_b200_decode with your own attn_logits",
                    need, (size_t)STATIC_WS_FLOATS);
    float *ws = nullptr;
    int rc = static_ws_address(&ws);
    if (rc) return rc;
    ommx_decode_args b = *a;
    b.attn_logits = ws;
    b.al_stride_s = (int64_t)row;
    b.al_stride_h = (int64_t)a->num_kv_splits * (int64_t)row;
    b.al_stride_b = (int64_t)a->n_q_heads * b.al_stride_h;
    rc = validate_decode(&b);
    if (rc) return rc;
    rc = launch_stage1(&b, (cudaStream_t)stream);
    if (rc) return rc;
    return launch_stage2(&b, (cudaStream_t)stream, true);
}

extern "C" int ommx_b200_merge_states(const float *o_parts, const float *lse_parts, const int32_t *valid_lens,
                                      int32_t P, int32_t R, int32_t D, float *o, float *lse, void *stream) {
    using namespace ommx;
    if (!o_parts || !lse_parts || !o || !lse) return fail(OMMX_E_ARG, "merge: null pointer");
    if (P < 0 || R < 0 || D <= 0) return fail(OMMX_E_ARG, "merge: P=%d R=%d D=%d", P, R, D);
    if (R == 0) return 0;
    merge_states_kernel<<<R, 128, 0, (cudaStream_t)stream>>>(o_parts, lse_parts, valid_lens, P, R, D, o, lse);
    OMMX_CUDA_TRY(cudaGetLastError());
    count_launch();
    return 0;
}

#ifdef OMMX_TRACE
// Development builds only: copy the probe array (32 warps x 256 slots of SM clock values) to the host.
extern "C" int ommx_b200_debug_read_trace(long long *host_out) {
    return cudaMemcpyFromSymbol(host_out, ommx::g_trace, sizeof(long long) * 32 * 256) == cudaSuccess ? 0 : OMMX_E_CUDA;
}
#endif
