// Decode GEMV (1 <= m <= 16) for GGML block-quantized weights on sm_100a.
//
// Computes the fused op behind compute.Function.FusedQuantizedDense
// (core/graph/fused_ops.go:195-245 in gomlx/gomlx):
//     y[m, n] = act(sum_k x[m, k] * dequant(W)[n, k] + bias[n])
//
// The kernel is bound by HBM, and the matrices of a decoder layer are small next to the
// machine (a 4096 x 14336 Q4_K matrix is 223 KB per SM), so what matters is how many
// bytes each SM has in flight.  Data movement:
//   * the packed weights live in 16-row x TK tiles whose bytes are contiguous (layout.cuh);
//     each warp streams its tiles with cp.async.bulk (the TMA unit, one instruction per
//     4.6-13 KB tile) into a private ring of shared-memory slots, completion tracked by one
//     mbarrier per slot.  Nearly the whole per-SM share of the matrix is requested at once;
//   * every packed byte is read from HBM exactly once;
//   * a CTA owns one K slice for its whole life, so its activations are staged once (as
//     fp16, in shared memory) and reused for all of its row tiles;
//   * the CTAs that hold the K slices of the same rows form a thread-block cluster and add
//     their partial sums through distributed shared memory in a fixed order (deterministic).
//
// Arithmetic: lanes read their 16-byte pieces of a tile with conflict-free LDS.128, unpack
// in registers and feed m16n8k16 tensor-core MMAs directly (A = 16 weight rows x 16 k,
// B = 16 k x 8 batch columns of activations, f32 accumulators).  Using the tensor cores
// keeps the instruction count per weight the same for m = 1 and m = 16.
//   * nibbles / bytes become fp16 through the exponent-magic trick (0x6400 | q is the
//     fp16 number 1024 + q), then one HFMA2 applies the block scale:
//     (1024 + q) * s - 1024 * s = q * s, exact before its single rounding;
//   * the constant offsets of the formats (-8 for Q4_0, -dmin*m for Q4_K, -32 for Q6_K)
//     are not applied per value.  They are linear in the per-sub-block sums of x, so
//     they are added by one extra MMA per tile whose A operand is the per-sub-block
//     coefficient (d, dmin*m, d*sc) and whose B operand is -offset * sum(x) of that
//     sub-block, split into an fp16 high and low part;
//   * Q8_0 is signed and needs no offset: (q + 128 + 1024) - 1152 is exact, then * d.
//
// Activations are rounded to fp16 (saturating at +-65504) when they are staged; weights are
// rounded to fp16 after scaling (block scales must stay below 64 in magnitude).
// Accumulation is f32.  Relative to the f32 reference this costs below 1e-3 of the output scale.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the kernel records a timeout in
// the status word and carries on, so a lost copy can never hang the GPU.
#include "common.cuh"

#include <cooperative_groups.h>

#include <algorithm>
#include <climits>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace cg = cooperative_groups;

namespace b200q {
namespace {

struct GemvParams {
    const uint8_t *tiles;
    const void *x;
    const float *bias;
    float *y;
    int *status;
    int64_t n, k, y_ld;
    int64_t rt, kt;
    int m, x_dtype, act;
    int ktc;     // k tiles per staged x chunk
    int splits;  // CTAs per cluster; split s owns k tiles [s*kts, (s+1)*kts)
    int kts;
    int nclusters;
    int depth;   // ring slots per warp
    int maxnj;   // upper bound on row tiles per warp
};

constexpr int kSpinLimit = 1 << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait; returns false if the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int spin = 0; spin < kSpinLimit; spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
// One TMA bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hfma2u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hsub2u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bcast_lo(uint32_t p) { return __byte_perm(p, p, 0x1010); }
__device__ __forceinline__ uint32_t bcast_hi(uint32_t p) { return __byte_perm(p, p, 0x3232); }

constexpr uint32_t H2_1024 = 0x64006400u;    // fp16x2 (1024, 1024)
constexpr uint32_t H2_N1024 = 0xE400E400u;   // (-1024, -1024)
constexpr uint32_t H2_N64 = 0xD400D400u;     // (-64, -64)
constexpr uint32_t H2_1152 = 0x64806480u;    // (1152, 1152)
constexpr uint32_t MAGIC_1024 = 0x64006400u; // exponent bits of 1024: low mantissa bits count 1
constexpr uint32_t MAGIC_64 = 0x54005400u;   // exponent bits of 64: mantissa bit 4 counts 1
constexpr uint32_t BYTES_64 = 0x64646464u;

// Two bytes of `v` (selected by `sel`) as the fp16 pair (1024 + b_lo, 1024 + b_hi).
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t v, uint32_t sel) { return __byte_perm(v, BYTES_64, sel); }
constexpr uint32_t SEL01 = 0x5140, SEL23 = 0x7362;

// Shared-memory addresses of the staged activations for the batch columns this lane feeds,
// already advanced to the current tile and to the lane's K-quarter.
//
// Staged x is stored in 16-byte chunks (8 fp16) whose index is XOR-ed with 2t (t = K-quarter of
// the chunk inside its tile), so that the four quarters a quad reads in one instruction fall
// into different banks.  For a chunk offset OFF that is known at compile time, OFF ^ 2t differs
// from OFF by +-2 (if t&1) and +-4 (if t&2) chunks with signs that depend only on OFF, so four
// pre-biased base addresses r[0..3] turn every load into `base + immediate`.
template <int NB>
struct XCols {
    uint32_t r[NB][4];  // x chunk bases: index = (bit1 of OFF) | (bit2 of OFF) << 1
    uint32_t shi[NB];   // aux sums (high part) of this lane's sub-blocks
    uint32_t slo[NB];   // aux sums (low part)
};

template <int NB>
struct XBase {
    uint32_t x[NB];    // staged row of the column, tile 0, quarter 0
    uint32_t shi[NB];
    uint32_t slo[NB];
};

template <int NB>
__device__ __forceinline__ void xcols_for_tile(XCols<NB> &xc, const XBase<NB> &xb, int chunk0, int sub0, int t) {
    const int a = (t & 1) * 32, b = (t >> 1) * 64;
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {
        const uint32_t base = xb.x[nb] + chunk0 * 16;
        xc.r[nb][0] = base + a + b;
        xc.r[nb][1] = base - a + b;
        xc.r[nb][2] = base + a - b;
        xc.r[nb][3] = base - a - b;
        xc.shi[nb] = xb.shi[nb] + sub0 * 2;
        xc.slo[nb] = xb.slo[nb] + sub0 * 2;
    }
}

// 8 staged activations of chunk OFF (relative to the lane's quarter of the current tile).
template <int NB>
__device__ __forceinline__ uint4 lds_chunk(const XCols<NB> &xc, int nb, int off) {
    return lds128(xc.r[nb][((off >> 1) & 1) | (((off >> 2) & 1) << 1)] + off * 16);
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// ---------------------------------------------------------------------------------------
// Q4_0 : tile = 16 rows x 512 k, 9 loads per lane.
// ---------------------------------------------------------------------------------------
template <int NB>
__device__ __forceinline__ void tile_q4_0(uint32_t slot, const XCols<NB> &xc, float (&acc)[2][NB][4]) {
    const uint4 sc = lds128(slot);
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {  // offset term: sum_b d_b * (-8 * sum(x in block b))
        const uint2 bh = lds64(xc.shi[nb]), bl = lds64(xc.slo[nb]);
        mma16816(acc[0][nb], sc.x, sc.z, sc.y, sc.w, bh.x, bh.y);
        mma16816(acc[1][nb], sc.x, sc.z, sc.y, sc.w, bl.x, bl.y);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t pg = i < 2 ? sc.x : sc.y, pg8 = i < 2 ? sc.z : sc.w;
        const uint32_t dg = (i & 1) ? bcast_hi(pg) : bcast_lo(pg), dg8 = (i & 1) ? bcast_hi(pg8) : bcast_lo(pg8);
        const uint32_t olo = hmul2u(dg, H2_N1024), ohi = hmul2u(dg, H2_N64);
        const uint32_t olo8 = hmul2u(dg8, H2_N1024), ohi8 = hmul2u(dg8, H2_N64);
        const uint4 qa = lds128(slot + (1 + 2 * i) * 512), qb = lds128(slot + (2 + 2 * i) * 512);
#pragma unroll
        for (int wp = 0; wp < 2; wp++) {
            uint4 blo[NB], bhi[NB];
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                blo[nb] = lds_chunk(xc, nb, 4 * i + wp);
                bhi[nb] = lds_chunk(xc, nb, 4 * i + 2 + wp);
            }
#pragma unroll
            for (int ww = 0; ww < 2; ww++) {
                const uint32_t wa = wp == 0 ? (ww == 0 ? qa.x : qa.y) : (ww == 0 ? qa.z : qa.w);
                const uint32_t wb = wp == 0 ? (ww == 0 ? qb.x : qb.y) : (ww == 0 ? qb.z : qb.w);
                const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
                const uint32_t l0 = hfma2u((wa & 0x000F000Fu) | MAGIC_1024, dg, olo);
                const uint32_t l1 = hfma2u((wb & 0x000F000Fu) | MAGIC_1024, dg8, olo8);
                const uint32_t l2 = hfma2u((wa8 & 0x000F000Fu) | MAGIC_1024, dg, olo);
                const uint32_t l3 = hfma2u((wb8 & 0x000F000Fu) | MAGIC_1024, dg8, olo8);
                const uint32_t h0 = hfma2u((wa & 0x00F000F0u) | MAGIC_64, dg, ohi);
                const uint32_t h1 = hfma2u((wb & 0x00F000F0u) | MAGIC_64, dg8, ohi8);
                const uint32_t h2 = hfma2u((wa8 & 0x00F000F0u) | MAGIC_64, dg, ohi);
                const uint32_t h3 = hfma2u((wb8 & 0x00F000F0u) | MAGIC_64, dg8, ohi8);
#pragma unroll
                for (int nb = 0; nb < NB; nb++) {
                    mma16816(acc[0][nb], l0, l1, l2, l3, ww == 0 ? blo[nb].x : blo[nb].z, ww == 0 ? blo[nb].y : blo[nb].w);
                    mma16816(acc[1][nb], h0, h1, h2, h3, ww == 0 ? bhi[nb].x : bhi[nb].z, ww == 0 ? bhi[nb].y : bhi[nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Q8_0 : tile = 16 rows x 512 k, 17 loads per lane.
// ---------------------------------------------------------------------------------------
template <int NB>
__device__ __forceinline__ void tile_q8_0(uint32_t slot, const XCols<NB> &xc, float (&acc)[2][NB][4]) {
    const uint4 sc = lds128(slot);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t pg = i < 2 ? sc.x : sc.y, pg8 = i < 2 ? sc.z : sc.w;
        const uint32_t dg = (i & 1) ? bcast_hi(pg) : bcast_lo(pg), dg8 = (i & 1) ? bcast_hi(pg8) : bcast_lo(pg8);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int j = 1 + 2 * (2 * i + h);
            const uint4 qa = lds128(slot + j * 512), qb = lds128(slot + (j + 1) * 512);
#pragma unroll
            for (int wp = 0; wp < 2; wp++) {
                uint4 b[NB];
#pragma unroll
                for (int nb = 0; nb < NB; nb++) b[nb] = lds_chunk(xc, nb, 4 * i + 2 * h + wp);
#pragma unroll
                for (int ww = 0; ww < 2; ww++) {
                    const uint32_t wa = (wp == 0 ? (ww == 0 ? qa.x : qa.y) : (ww == 0 ? qa.z : qa.w)) ^ 0x80808080u;
                    const uint32_t wb = (wp == 0 ? (ww == 0 ? qb.x : qb.y) : (ww == 0 ? qb.z : qb.w)) ^ 0x80808080u;
                    const uint32_t a0 = hmul2u(hsub2u(bytes_to_h2(wa, SEL01), H2_1152), dg);
                    const uint32_t a1 = hmul2u(hsub2u(bytes_to_h2(wb, SEL01), H2_1152), dg8);
                    const uint32_t a2 = hmul2u(hsub2u(bytes_to_h2(wa, SEL23), H2_1152), dg);
                    const uint32_t a3 = hmul2u(hsub2u(bytes_to_h2(wb, SEL23), H2_1152), dg8);
#pragma unroll
                    for (int nb = 0; nb < NB; nb++)
                        mma16816(acc[ww][nb], a0, a1, a2, a3, ww == 0 ? b[nb].x : b[nb].z, ww == 0 ? b[nb].y : b[nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Q4_K : tile = 16 rows x 1024 k (4 super-blocks, one per quad lane), 18 loads per lane.
// ---------------------------------------------------------------------------------------
// Header (d, dmin, scales[12]) -> fp16 pairs ds[j/2] = d*sc_j and cm[j/2] = dmin*m_j.
__device__ __forceinline__ void q4k_header(const uint4 &h, uint32_t (&ds)[4], uint32_t (&cm)[4]) {
    const uint32_t d2 = bcast_lo(h.x), dmin2 = bcast_hi(h.x);
    const uint32_t sc0 = h.y & 0x3F3F3F3Fu, m0 = h.z & 0x3F3F3F3Fu;
    const uint32_t sc1 = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    const uint32_t m1 = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    ds[0] = hmul2u(hsub2u(bytes_to_h2(sc0, SEL01), H2_1024), d2);
    ds[1] = hmul2u(hsub2u(bytes_to_h2(sc0, SEL23), H2_1024), d2);
    ds[2] = hmul2u(hsub2u(bytes_to_h2(sc1, SEL01), H2_1024), d2);
    ds[3] = hmul2u(hsub2u(bytes_to_h2(sc1, SEL23), H2_1024), d2);
    cm[0] = hmul2u(hsub2u(bytes_to_h2(m0, SEL01), H2_1024), dmin2);
    cm[1] = hmul2u(hsub2u(bytes_to_h2(m0, SEL23), H2_1024), dmin2);
    cm[2] = hmul2u(hsub2u(bytes_to_h2(m1, SEL01), H2_1024), dmin2);
    cm[3] = hmul2u(hsub2u(bytes_to_h2(m1, SEL23), H2_1024), dmin2);
}

template <int NB>
__device__ __forceinline__ void tile_q4_k(uint32_t slot, const XCols<NB> &xc, float (&acc)[2][NB][4]) {
    uint32_t dsA[4], cmA[4], dsB[4], cmB[4];
    q4k_header(lds128(slot), dsA, cmA);
    q4k_header(lds128(slot + 512), dsB, cmB);
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {  // offset term: sum_j (dmin*m_j) * (-sum(x in sub-block j))
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const uint2 bh = lds64(xc.shi[nb] + 8 * q), bl = lds64(xc.slo[nb] + 8 * q);
            mma16816(acc[0][nb], cmA[2 * q], cmB[2 * q], cmA[2 * q + 1], cmB[2 * q + 1], bh.x, bh.y);
            mma16816(acc[1][nb], cmA[2 * q], cmB[2 * q], cmA[2 * q + 1], cmB[2 * q + 1], bl.x, bl.y);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int G = i >> 1, hf = i & 1;
        // low nibbles: sub-block 2G (low half of pair G); high nibbles: sub-block 2G+1.
        const uint32_t sl = bcast_lo(dsA[G]), sh = bcast_hi(dsA[G]), sl8 = bcast_lo(dsB[G]), sh8 = bcast_hi(dsB[G]);
        const uint32_t olo = hmul2u(sl, H2_N1024), ohi = hmul2u(sh, H2_N64);
        const uint32_t olo8 = hmul2u(sl8, H2_N1024), ohi8 = hmul2u(sh8, H2_N64);
        const uint4 qa = lds128(slot + (2 + 2 * i) * 512), qb = lds128(slot + (3 + 2 * i) * 512);
#pragma unroll
        for (int wp = 0; wp < 2; wp++) {
            uint4 blo[NB], bhi[NB];
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                blo[nb] = lds_chunk(xc, nb, 8 * G + 2 * hf + wp);
                bhi[nb] = lds_chunk(xc, nb, 8 * G + 2 * hf + 4 + wp);
            }
#pragma unroll
            for (int ww = 0; ww < 2; ww++) {
                const uint32_t wa = wp == 0 ? (ww == 0 ? qa.x : qa.y) : (ww == 0 ? qa.z : qa.w);
                const uint32_t wb = wp == 0 ? (ww == 0 ? qb.x : qb.y) : (ww == 0 ? qb.z : qb.w);
                const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
                const uint32_t l0 = hfma2u((wa & 0x000F000Fu) | MAGIC_1024, sl, olo);
                const uint32_t l1 = hfma2u((wb & 0x000F000Fu) | MAGIC_1024, sl8, olo8);
                const uint32_t l2 = hfma2u((wa8 & 0x000F000Fu) | MAGIC_1024, sl, olo);
                const uint32_t l3 = hfma2u((wb8 & 0x000F000Fu) | MAGIC_1024, sl8, olo8);
                const uint32_t h0 = hfma2u((wa & 0x00F000F0u) | MAGIC_64, sh, ohi);
                const uint32_t h1 = hfma2u((wb & 0x00F000F0u) | MAGIC_64, sh8, ohi8);
                const uint32_t h2 = hfma2u((wa8 & 0x00F000F0u) | MAGIC_64, sh, ohi);
                const uint32_t h3 = hfma2u((wb8 & 0x00F000F0u) | MAGIC_64, sh8, ohi8);
#pragma unroll
                for (int nb = 0; nb < NB; nb++) {
                    mma16816(acc[0][nb], l0, l1, l2, l3, ww == 0 ? blo[nb].x : blo[nb].z, ww == 0 ? blo[nb].y : blo[nb].w);
                    mma16816(acc[1][nb], h0, h1, h2, h3, ww == 0 ? bhi[nb].x : bhi[nb].z, ww == 0 ? bhi[nb].y : bhi[nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Q6_K : tile = 16 rows x 1024 k (4 super-blocks), 26 loads + one 4-byte load per lane.
// ---------------------------------------------------------------------------------------
// int8 scales[16] and d -> fp16 pairs ds[s/2] = d * sc_s.
__device__ __forceinline__ void q6k_scales(const uint4 &s, uint32_t d2, uint32_t (&ds)[8]) {
    const uint32_t w[4] = {s.x ^ 0x80808080u, s.y ^ 0x80808080u, s.z ^ 0x80808080u, s.w ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        ds[2 * i] = hmul2u(hsub2u(bytes_to_h2(w[i], SEL01), H2_1152), d2);
        ds[2 * i + 1] = hmul2u(hsub2u(bytes_to_h2(w[i], SEL23), H2_1152), d2);
    }
}

template <int NB>
__device__ __forceinline__ void tile_q6_k(uint32_t slot, uint32_t slot_tail, const XCols<NB> &xc,
                                          float (&acc)[2][NB][4]) {
    uint32_t dsA[8], dsB[8];
    const uint32_t tail = lds32(slot_tail);  // fp16 d of row g | row g+8
    q6k_scales(lds128(slot), bcast_lo(tail), dsA);
    q6k_scales(lds128(slot + 512), bcast_hi(tail), dsB);
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {  // offset term: sum_s (d*sc_s) * (-32 * sum(x in sub-block s))
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint2 bh = lds64(xc.shi[nb] + 8 * q), bl = lds64(xc.slo[nb] + 8 * q);
            mma16816(acc[0][nb], dsA[2 * q], dsB[2 * q], dsA[2 * q + 1], dsB[2 * q + 1], bh.x, bh.y);
            mma16816(acc[1][nb], dsA[2 * q], dsB[2 * q], dsA[2 * q + 1], dsB[2 * q + 1], bl.x, bl.y);
        }
    }
#pragma unroll
    for (int gr = 0; gr < 4; gr++) {
        const int n = gr >> 1, lh = gr & 1, j0 = 2 + 6 * gr;
        const uint4 la = lds128(slot + j0 * 512), la8 = lds128(slot + (j0 + 1) * 512), lb = lds128(slot + (j0 + 2) * 512),
                    lb8 = lds128(slot + (j0 + 3) * 512), hh = lds128(slot + (j0 + 4) * 512),
                    hh8 = lds128(slot + (j0 + 5) * 512);
        uint32_t s[4], s8[4], o[4], o8[4];
#pragma unroll
        for (int c = 0; c < 4; c++) {  // code c uses scale 8n + lh + 2c = half lh of pair 4n + c
            s[c] = lh ? bcast_hi(dsA[4 * n + c]) : bcast_lo(dsA[4 * n + c]);
            s8[c] = lh ? bcast_hi(dsB[4 * n + c]) : bcast_lo(dsB[4 * n + c]);
            o[c] = hmul2u(s[c], H2_N1024);
            o8[c] = hmul2u(s8[c], H2_N1024);
        }
#pragma unroll
        for (int wp = 0; wp < 2; wp++) {
            uint4 b[4][NB];
#pragma unroll
            for (int c = 0; c < 4; c++)
#pragma unroll
                for (int nb = 0; nb < NB; nb++) b[c][nb] = lds_chunk(xc, nb, 16 * n + 2 * lh + 4 * c + wp);
#pragma unroll
            for (int ww = 0; ww < 2; ww++) {
                const uint32_t a = wp == 0 ? (ww == 0 ? la.x : la.y) : (ww == 0 ? la.z : la.w);
                const uint32_t a8 = wp == 0 ? (ww == 0 ? la8.x : la8.y) : (ww == 0 ? la8.z : la8.w);
                const uint32_t bq = wp == 0 ? (ww == 0 ? lb.x : lb.y) : (ww == 0 ? lb.z : lb.w);
                const uint32_t bq8 = wp == 0 ? (ww == 0 ? lb8.x : lb8.y) : (ww == 0 ? lb8.z : lb8.w);
                const uint32_t h = wp == 0 ? (ww == 0 ? hh.x : hh.y) : (ww == 0 ? hh.z : hh.w);
                const uint32_t h8 = wp == 0 ? (ww == 0 ? hh8.x : hh8.y) : (ww == 0 ? hh8.z : hh8.w);
                uint32_t code[4], code8[4];
                code[0] = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
                code[1] = (bq & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
                code[2] = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
                code[3] = ((bq >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
                code8[0] = (a8 & 0x0F0F0F0Fu) | ((h8 << 4) & 0x30303030u);
                code8[1] = (bq8 & 0x0F0F0F0Fu) | ((h8 << 2) & 0x30303030u);
                code8[2] = ((a8 >> 4) & 0x0F0F0F0Fu) | (h8 & 0x30303030u);
                code8[3] = ((bq8 >> 4) & 0x0F0F0F0Fu) | ((h8 >> 2) & 0x30303030u);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint32_t a0 = hfma2u(bytes_to_h2(code[c], SEL01), s[c], o[c]);
                    const uint32_t a1 = hfma2u(bytes_to_h2(code8[c], SEL01), s8[c], o8[c]);
                    const uint32_t a2 = hfma2u(bytes_to_h2(code[c], SEL23), s[c], o[c]);
                    const uint32_t a3 = hfma2u(bytes_to_h2(code8[c], SEL23), s8[c], o8[c]);
#pragma unroll
                    for (int nb = 0; nb < NB; nb++)
                        mma16816(acc[c & 1][nb], a0, a1, a2, a3, ww == 0 ? b[c][nb].x : b[c][nb].z,
                                 ww == 0 ? b[c][nb].y : b[c][nb].w);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Activation staging: x[m, k0 .. k0+kc) -> fp16 in shared memory, plus the per-sub-block
// sums needed by the offset MMAs.  One thread handles 8 consecutive values.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f2h2_sat(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

template <int TYPE>
__device__ __forceinline__ void stage_x(const GemvParams &p, int64_t k0, int kc, int xs_stride, int ns, __half *xs,
                                        __half *shi, __half *slo) {
    using F = Fmt<TYPE>;
    const int gpc = kc >> 3;  // 8-value groups per column, a multiple of 64
    const int total = p.m * gpc;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int col = idx / gpc, gi = idx - col * gpc;
        const int64_t k = k0 + (int64_t)gi * 8;
        float v[8];
        if (k < p.k) {
            if (p.x_dtype == B200Q_F32) {
                const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(p.x) + col * p.k + k);
                const float4 a = __ldg(src), b = __ldg(src + 1);
                v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
            } else {
                const uint4 r =
                    __ldg(reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.x) + col * p.k + k));
                const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    v[2 * i] = __uint_as_float(w[i] << 16);
                    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.0f;
        }
        uint4 out;
        if constexpr (F::PERM4) {
            out.x = f2h2_sat(v[0], v[2]), out.y = f2h2_sat(v[1], v[3]);
            out.z = f2h2_sat(v[4], v[6]), out.w = f2h2_sat(v[5], v[7]);
        } else {
            out.x = f2h2_sat(v[0], v[1]), out.y = f2h2_sat(v[2], v[3]);
            out.z = f2h2_sat(v[4], v[5]), out.w = f2h2_sat(v[6], v[7]);
        }
        const int tq = ((gi << 3) & (F::TK - 1)) / (F::TK / 4);
        *reinterpret_cast<uint4 *>(xs + col * xs_stride + ((gi ^ (2 * tq)) << 3)) = out;
        if constexpr (F::SUB != 0) {
            // Sums are taken over the rounded values the MMAs will see, so the offset cancels exactly.
            const uint32_t w[4] = {out.x, out.y, out.z, out.w};
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                sum += f.x + f.y;
            }
            constexpr float OFFSET = TYPE == kQ4_0 ? 8.0f : TYPE == kQ4_K ? 1.0f : 32.0f;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if constexpr (F::SUB == 32) sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            constexpr int GPS = F::SUB / 8;  // groups per sub-block
            if ((gi & (GPS - 1)) == 0) {
                const float s = -OFFSET * sum;
                const __half hi = __float2half_rn(s);
                const __half lo = __float2half_rn(s - __half2float(hi));
                shi[col * ns + gi / GPS] = hi;
                slo[col * ns + gi / GPS] = lo;
            }
        }
    }
}

// Walks one warp's tile sequence: x chunks (outer), the warp's row tiles (middle), k tiles (inner).
struct TileWalk {
    int64_t kt0;
    int j, kl;
};

// Grid = nclusters x splits CTAs; the `splits` CTAs of a cluster hold the K slices of the same rows.
// Cluster c owns row tiles [c*RT/nclusters, (c+1)*RT/nclusters); inside a CTA warp w takes every
// nwarps-th of them.  Shared memory: staged x | aux sums | partial sums | tile rings | mbarriers.
template <int TYPE, int NB>
__global__ void __launch_bounds__(512, 1) gemv_mma_kernel(const GemvParams p) {
    using F = Fmt<TYPE>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nwarps = blockDim.x >> 5;
    const int kc_max = p.ktc * F::TK;
    const int xs_stride = kc_max + 8;
    const int ns = F::SUB ? kc_max / F::SUB : 0;
    size_t off = 0;
    __half *xs = reinterpret_cast<__half *>(smem);
    off += (size_t)p.m * xs_stride * 2;
    __half *shi = reinterpret_cast<__half *>(smem + off);
    __half *slo = shi + (size_t)p.m * ns;
    off += (size_t)p.m * ns * 4;
    off = (off + 15) & ~(size_t)15;
    float *red = reinterpret_cast<float *>(smem + off);  // [j][warp][nb][i][lane]
    off += (size_t)p.maxnj * nwarps * NB * 128 * sizeof(float);
    off = (off + 127) & ~(size_t)127;
    uint8_t *ring = smem + off + (size_t)warp * p.depth * F::TILE;
    off += (size_t)nwarps * p.depth * F::TILE;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + off) + warp * p.depth;

    const int split = (int)(blockIdx.x % p.splits);
    const int64_t cl = blockIdx.x / p.splits;
    const int64_t r0 = cl * p.rt / p.nclusters, r1 = (cl + 1) * p.rt / p.nclusters;
    const int64_t kt_begin = (int64_t)split * p.kts, kt_end = min(kt_begin + p.kts, p.kt);
    const int nj = (kt_begin < kt_end && r0 + warp < r1) ? (int)((r1 - r0 - warp + nwarps - 1) / nwarps) : 0;
    const int total = nj * (int)(kt_end > kt_begin ? kt_end - kt_begin : 0);  // tiles this warp consumes

    const uint32_t ring_s = smem_u32(ring), bars_s = smem_u32(bars);
    if (lane == 0) {
        for (int d = 0; d < p.depth; d++) mbar_init(bars_s + 8 * d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // Producer side (lane 0 of each warp): request the next tile of the warp's sequence into ring
    // slot `pd`.  Sequence order: x chunks (outer), the warp's row tiles, k tiles of the chunk.
    TileWalk pw{kt_begin, 0, 0};
    int issued = 0, pd = 0;
    auto issue_next = [&]() {
        const int nkt = (int)min((int64_t)p.ktc, kt_end - pw.kt0);
        const int64_t rt = r0 + warp + (int64_t)pw.j * nwarps;
        const uint8_t *src = p.tiles + (rt * p.kt + pw.kt0 + pw.kl) * (int64_t)F::TILE;
        mbar_expect_tx(bars_s + 8 * pd, F::TILE);
        bulk_load(ring_s + pd * F::TILE, src, F::TILE, bars_s + 8 * pd);
        issued++;
        if (++pd == p.depth) pd = 0;
        if (++pw.kl == nkt) {
            pw.kl = 0;
            if (++pw.j == nj) {
                pw.j = 0;
                pw.kt0 += p.ktc;
            }
        }
    };
    if (lane == 0)
        while (issued < total && issued < p.depth) issue_next();

    XBase<NB> xb;
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {
        const int col = min(g + 8 * nb, p.m - 1);
        // the lane's K-quarter t starts TK/4 values = TK/32 chunks into each tile
        xb.x[nb] = smem_u32(xs + col * xs_stride) + t * (F::TK / 32) * 16;
        if constexpr (F::SUB != 0) {
            // the lane's sub-blocks start (TK/4)/SUB entries into each tile's aux range
            xb.shi[nb] = smem_u32(shi + col * ns) + t * (F::TK / 4 / F::SUB) * 2;
            xb.slo[nb] = smem_u32(slo + col * ns) + t * (F::TK / 4 / F::SUB) * 2;
        } else {
            xb.shi[nb] = xb.slo[nb] = 0;
        }
    }

    int cd = 0;
    uint32_t cphase = 0;
    bool timed_out = false;
    for (int64_t kt0 = kt_begin; kt0 < kt_end; kt0 += p.ktc) {
        const int nkt = (int)min((int64_t)p.ktc, kt_end - kt0);
        if (kt0 != kt_begin) __syncthreads();  // everyone is done reading the previous chunk
        stage_x<TYPE>(p, kt0 * F::TK, nkt * F::TK, xs_stride, ns, xs, shi, slo);
        __syncthreads();
        for (int j = 0; j < nj; j++) {
            float acc[2][NB][4];
#pragma unroll
            for (int a = 0; a < 2; a++)
#pragma unroll
                for (int nb = 0; nb < NB; nb++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[a][nb][i] = 0.0f;
            for (int kl = 0; kl < nkt; kl++) {
                if (!mbar_wait(bars_s + 8 * cd, cphase)) timed_out = true;
                const uint32_t slot = ring_s + cd * F::TILE + lane * 16;
                XCols<NB> xc;
                xcols_for_tile<NB>(xc, xb, kl * (F::TK / 8), F::SUB ? kl * (F::TK / F::SUB) : 0, t);
                if constexpr (TYPE == kQ4_0) {
                    tile_q4_0<NB>(slot, xc, acc);
                } else if constexpr (TYPE == kQ8_0) {
                    tile_q8_0<NB>(slot, xc, acc);
                } else if constexpr (TYPE == kQ4_K) {
                    tile_q4_k<NB>(slot, xc, acc);
                } else {
                    tile_q6_k<NB>(slot, ring_s + cd * F::TILE + F::LOADS * 512 + lane * 4, xc, acc);
                }
                if (++cd == p.depth) cd = 0, cphase ^= 1;
                __syncwarp();  // all lanes have read the slot
                if (lane == 0 && issued < total) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    issue_next();
                }
            }
            // Park the partial sums of this row tile; later chunks of the same K slice add to them.
            float *r = red + (size_t)(j * nwarps + warp) * NB * 128 + lane;
#pragma unroll
            for (int nb = 0; nb < NB; nb++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float *q = r + (nb * 4 + i) * 32;
                    const float v = acc[0][nb][i] + acc[1][nb][i];
                    *q = (kt0 == kt_begin) ? v : *q + v;
                }
        }
    }
    if (timed_out && lane == 0) atomicExch(p.status, 2);

    cg::cluster_group cluster = cg::this_cluster();
    if (p.splits > 1) cluster.sync(); else __syncthreads();

    // Element e of `red`: lane = e & 31, i = (e >> 5) & 3, nb, warp, j.  D fragment element i of lane
    // (g, t): row g + 8*(i>>1) of the row tile, batch column 2t + (i&1) + 8*nb.
    const int maxnj_cl = (int)((r1 - r0 + nwarps - 1) / nwarps);
    const int total_e = maxnj_cl * nwarps * NB * 128;
    const int per = (total_e + p.splits - 1) / p.splits;
    const int e_end = min((split + 1) * per, total_e);
    for (int e = split * per + (int)threadIdx.x; e < e_end; e += blockDim.x) {
        const int ln = e & 31, i = (e >> 5) & 3, nb = (e >> 7) % NB, wj = (e >> 7) / NB;
        const int wq = wj % nwarps, j = wj / nwarps;
        const int64_t rtile = r0 + wq + (int64_t)j * nwarps;
        const int64_t row = rtile * 16 + (ln >> 2) + 8 * (i >> 1);
        const int col = 8 * nb + 2 * (ln & 3) + (i & 1);
        if (rtile < r1 && row < p.n && col < p.m) {
            float v = 0.0f;
            if (p.splits > 1) {
                for (int r = 0; r < p.splits; r++) {
                    // a split whose K slice is empty parked nothing
                    if ((int64_t)r * p.kts < p.kt) v += *cluster.map_shared_rank(red + e, r);
                }
            } else {
                v = red[e];
            }
            if (p.bias != nullptr) v += __ldg(p.bias + row);
            p.y[(int64_t)col * p.y_ld + row] = apply_activation(p.act, v);
        }
    }
    if (p.splits > 1) cluster.sync();  // keep shared memory alive until every peer has read it
}

int env_int(const char *name, int dflt) {
    const char *v = std::getenv(name);
    return v && *v ? std::atoi(v) : dflt;
}

constexpr size_t kSmemLimit = 227 * 1024;
constexpr int kMaxWarps = 16;

template <int TYPE, int NB>
int launch_t(const Weight &w, const GemvParams &p0, cudaStream_t s) {
    using F = Fmt<TYPE>;
    GemvParams p = p0;
    int dev_sms = 148;
    cudaDeviceGetAttribute(&dev_sms, cudaDevAttrMultiProcessorCount, w.device);

    // K splits (CTAs per cluster).  Two halves of K per row group measured best for every decoder
    // shape on B200; matrices with few rows (N <= 16 * #SMs) need four to give all SMs work.
    int splits = w.kt >= 2 ? 2 : 1;
    if (w.rt <= dev_sms && w.kt >= 4) splits = 4;
    if (w.kt % splits != 0)  // prefer an even split when one exists nearby
        for (int sp = splits; sp <= 8 && sp <= w.kt; sp++)
            if (w.kt % sp == 0) { splits = sp; break; }
    splits = std::max(1, std::min(8, env_int("B200Q_GEMV_SPLITS", splits)));
    splits = (int)std::min<int64_t>(splits, w.kt);
    p.splits = splits;
    p.kts = (int)((w.kt + splits - 1) / splits);

    // One cluster per `splits` SMs, but never more clusters than row tiles.
    int nclusters = std::max(1, dev_sms / splits);
    nclusters = env_int("B200Q_GEMV_CLUSTERS", nclusters);
    nclusters = (int)std::max<int64_t>(1, std::min<int64_t>(nclusters, w.rt));
    p.nclusters = nclusters;
    const int64_t rows_per_cluster = (w.rt + nclusters - 1) / nclusters;

    // Staged x chunk: as much of the K slice as fits the x budget.
    const size_t per_tile_x = (size_t)p.m * (F::TK * 2 + (F::SUB ? 4 * (F::TK / F::SUB) : 0));
    const size_t x_budget = (size_t)env_int("B200Q_GEMV_XSMEM", 48 * 1024);
    const int ktc = (int)std::max<size_t>(1, std::min<size_t>((x_budget - p.m * 16) / per_tile_x, p.kts));
    p.ktc = ktc;
    const size_t x_bytes =
        (((size_t)p.m * (ktc * F::TK + 8) * 2 + (F::SUB ? (size_t)p.m * (ktc * F::TK / F::SUB) * 4 : 0)) + 15) & ~(size_t)15;

    // Warps per CTA: each warp walks whole row tiles, so prefer the count that needs the fewest
    // rounds and wastes the fewest warp-slots in the last round; then shrink until the per-warp
    // tile rings (at least two slots each, if possible) fit in shared memory next to x.
    int warps = 1;
    {
        int64_t best = INT64_MAX;
        for (int wc = 1; wc <= kMaxWarps; wc++) {
            const int64_t rounds = (rows_per_cluster + wc - 1) / wc;
            const int64_t cost = rounds * 64 + (rounds * wc - rows_per_cluster);  // time first, waste second
            if (cost <= best) best = cost, warps = wc;
        }
    }
    warps = std::max(1, std::min(kMaxWarps, env_int("B200Q_GEMV_WARPS", warps)));
    size_t fixed = 0, bar_bytes = 0;
    int depth = 0;
    for (;; warps--) {
        p.maxnj = (int)((rows_per_cluster + warps - 1) / warps);
        const size_t red_bytes = (size_t)p.maxnj * warps * NB * 128 * sizeof(float);
        fixed = (x_bytes + red_bytes + 127) & ~(size_t)127;
        bar_bytes = (size_t)warps * 8 * 8;  // depth <= 8
        depth = fixed + bar_bytes < kSmemLimit ? (int)((kSmemLimit - fixed - bar_bytes) / ((size_t)warps * F::TILE)) : 0;
        if (depth >= 2 || warps == 1) break;
    }
    if (depth < 1) return fail(B200Q_EINVAL, "gemv: shared memory budget exceeded for this shape");
    const int64_t tiles_per_warp = (int64_t)p.maxnj * p.kts;
    depth = (int)std::max<int64_t>(1, std::min<int64_t>({(int64_t)depth, (int64_t)8, tiles_per_warp}));
    depth = std::max(1, std::min(depth, env_int("B200Q_GEMV_DEPTH", depth)));
    p.depth = depth;
    const size_t smem = fixed + (size_t)warps * depth * F::TILE + (size_t)warps * depth * 8;

    auto kern = gemv_mma_kernel<TYPE, NB>;
    static thread_local bool configured[16] = {};
    if (!configured[w.device & 15]) {
        B200Q_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit));
        configured[w.device & 15] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(nclusters * splits), 1, 1);
    cfg.blockDim = dim3(warps * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200Q_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return 0;
}

template <int TYPE>
int launch_nb(const Weight &w, const GemvParams &p, cudaStream_t s) {
    return p.m <= 8 ? launch_t<TYPE, 1>(w, p, s) : launch_t<TYPE, 2>(w, p, s);
}

}  // namespace

int launch_gemv(const Weight &w, const void *x, int x_dtype, int m, const float *bias, int act, float *y, int64_t y_ld,
                cudaStream_t s) {
    if (m < 1 || m > 16) return fail(B200Q_EINVAL, "gemv: m must be in 1..16");
    GemvParams p{};
    p.tiles = w.tiles;
    p.x = x;
    p.bias = bias;
    p.y = y;
    p.n = w.n, p.k = w.k, p.y_ld = y_ld;
    p.rt = w.rt, p.kt = w.kt;
    p.m = m, p.x_dtype = x_dtype, p.act = act;
    p.status = w.status;
    switch (w.type) {
    case kQ4_0: return launch_nb<kQ4_0>(w, p, s);
    case kQ8_0: return launch_nb<kQ8_0>(w, p, s);
    case kQ4_K: return launch_nb<kQ4_K>(w, p, s);
    case kQ6_K: return launch_nb<kQ6_K>(w, p, s);
    }
    return fail(B200Q_ENOTIMPL, "gemv: unsupported GGML type");
}

}  // namespace b200q
