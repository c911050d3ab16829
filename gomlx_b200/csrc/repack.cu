// Upload-time rearrangement into the lane-tile layout, and the two consumers that
// need exact f32 values: ggml.Dequantize (ml/ggml/dequant.go:39-115 in gomlx/gomlx)
// and the embedding lookup (ml/ggml/gather.go:21-49).  Every f32 operation below is a
// single correctly rounded multiply / subtract (no FMA contraction), in the order the
// reference uses, so the results are bit-identical to a scalar CPU evaluation.
#include "common.cuh"

namespace b200q {

template <int TYPE>
__global__ void repack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int64_t n, int64_t k,
                              int64_t rt_count, int64_t kt_count) {
    using F = Fmt<TYPE>;
    constexpr int BPT = F::TK / F::VPB;  // blocks per tile along K
    const int64_t blocks_per_row = kt_count * BPT;
    const int64_t total = rt_count * 16 * blocks_per_row;
    const int64_t src_blocks_per_row = k / F::VPB;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / blocks_per_row, blk = idx % blocks_per_row;
        const int64_t rt = row >> 4, kt = blk / BPT;
        const int r = (int)(row & 15), b = (int)(blk % BPT);
        uint8_t *tile = dst + (rt * kt_count + kt) * (int64_t)F::TILE;
        const bool valid = row < n && blk < src_blocks_per_row;
        const uint16_t *s = reinterpret_cast<const uint16_t *>(src + (row * src_blocks_per_row + blk) * F::BPB);
#pragma unroll 1
        for (int o = 0; o < F::BPB; o += 2) {
            const uint16_t v = valid ? s[o >> 1] : (uint16_t)0;
            *reinterpret_cast<uint16_t *>(tile + tile_byte_offset<TYPE>(r, b, o)) = v;
        }
    }
}

// Reassembles the native bytes of one block from the tile.
template <int TYPE>
__device__ __forceinline__ void fetch_block(const uint8_t *tiles, int64_t kt_count, int64_t row, int64_t blk,
                                            uint16_t *out /* BPB/2 */) {
    using F = Fmt<TYPE>;
    constexpr int BPT = F::TK / F::VPB;
    const uint8_t *tile = tiles + ((row >> 4) * kt_count + blk / BPT) * (int64_t)F::TILE;
    const int r = (int)(row & 15), b = (int)(blk % BPT);
#pragma unroll 1
    for (int o = 0; o < F::BPB; o += 2)
        out[o >> 1] = *reinterpret_cast<const uint16_t *>(tile + tile_byte_offset<TYPE>(r, b, o));
}

__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

// Exact dequantization of one block into out[0..VPB).
template <int TYPE>
__device__ __forceinline__ void dequant_block(const uint16_t *blk16, float *out) {
    const uint8_t *blk = reinterpret_cast<const uint8_t *>(blk16);
    if constexpr (TYPE == kQ8_0) {  // dequant.go:58-78
        const float d = h2f(blk16[0]);
        for (int i = 0; i < 32; i++) out[i] = __fmul_rn((float)(int8_t)blk[2 + i], d);
    } else if constexpr (TYPE == kQ4_0) {  // dequant.go:83-115
        const float d = h2f(blk16[0]);
        for (int j = 0; j < 16; j++) {
            const uint8_t q = blk[2 + j];
            out[j] = __fmul_rn(__fsub_rn((float)(q & 0x0f), 8.0f), d);
            out[16 + j] = __fmul_rn(__fsub_rn((float)(q >> 4), 8.0f), d);
        }
    } else if constexpr (TYPE == kQ4_K) {
        const float d = h2f(blk16[0]), dmin = h2f(blk16[1]);
        const uint8_t *s = blk + 4, *qs = blk + 16;
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            if (j < 4) {
                sc = s[j] & 63;
                m = s[j + 4] & 63;
            } else {
                sc = (uint8_t)((s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4));
                m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
            }
            const float ds = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)m);
            const int gq = j >> 1, hi = j & 1;
            for (int l = 0; l < 32; l++) {
                const uint8_t q = qs[32 * gq + l];
                out[32 * j + l] = __fsub_rn(__fmul_rn(ds, (float)(hi ? (q >> 4) : (q & 0x0f))), dm);
            }
        }
    } else {  // Q6_K
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192);
        const float d = h2f(blk16[104]);
        for (int n = 0; n < 2; n++)
            for (int l = 0; l < 32; l++) {
                const int is = 8 * n + l / 16;
                const uint8_t h = qh[32 * n + l];
                const int q1 = (int)((ql[64 * n + l] & 0x0f) | (((h >> 0) & 3) << 4)) - 32;
                const int q2 = (int)((ql[64 * n + 32 + l] & 0x0f) | (((h >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((ql[64 * n + l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((ql[64 * n + 32 + l] >> 4) | (((h >> 6) & 3) << 4)) - 32;
                out[128 * n + l] = __fmul_rn(__fmul_rn(d, (float)sc[is + 0]), (float)q1);
                out[128 * n + 32 + l] = __fmul_rn(__fmul_rn(d, (float)sc[is + 2]), (float)q2);
                out[128 * n + 64 + l] = __fmul_rn(__fmul_rn(d, (float)sc[is + 4]), (float)q3);
                out[128 * n + 96 + l] = __fmul_rn(__fmul_rn(d, (float)sc[is + 6]), (float)q4);
            }
    }
}

// One thread per (output row, block).  `idx` == nullptr: row i of the output is row i of
// the weight (Dequantize); otherwise row i of the output is table row idx[i] (gather).
template <int TYPE>
__global__ void dequant_rows_kernel(const uint8_t *__restrict__ tiles, int64_t n, int64_t k, int64_t kt_count,
                                    const int32_t *__restrict__ idx, int64_t n_out, float *__restrict__ out,
                                    int *__restrict__ status) {
    using F = Fmt<TYPE>;
    const int64_t bpr = k / F::VPB;
    const int64_t total = n_out * bpr;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t orow = i / bpr, blk = i % bpr;
        int64_t row = orow;
        if (idx != nullptr) {
            row = idx[orow];
            if (row < 0 || row >= n) {  // report, write zeros, touch nothing out of range
                if (blk == 0) atomicExch(status, 1);
                float *o = out + orow * k + blk * F::VPB;
                for (int e = 0; e < F::VPB; e++) o[e] = 0.0f;
                continue;
            }
        }
        uint16_t raw[F::BPB / 2];
        fetch_block<TYPE>(tiles, kt_count, row, blk, raw);
        dequant_block<TYPE>(raw, out + orow * k + blk * F::VPB);
    }
}

template <int TYPE>
static int repack_t(const Weight &w, const uint8_t *src, cudaStream_t s) {
    const int64_t total = w.rt * 16 * w.kt * (Fmt<TYPE>::TK / Fmt<TYPE>::VPB);
    const int threads = 256;
    const int64_t blocks = (total + threads - 1) / threads;
    repack_kernel<TYPE><<<(unsigned)(blocks > 65535 * 16 ? 65535 * 16 : blocks), threads, 0, s>>>(src, w.tiles, w.n, w.k,
                                                                                                 w.rt, w.kt);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, "repack launch");
}

int launch_repack(const Weight &w, const uint8_t *src, cudaStream_t s) {
    switch (w.type) {
    case kQ4_0: return repack_t<kQ4_0>(w, src, s);
    case kQ8_0: return repack_t<kQ8_0>(w, src, s);
    case kQ4_K: return repack_t<kQ4_K>(w, src, s);
    case kQ6_K: return repack_t<kQ6_K>(w, src, s);
    }
    return fail(B200Q_ENOTIMPL, "repack: unsupported GGML type");
}

template <int TYPE>
static int dequant_t(const Weight &w, const int32_t *idx, int64_t n_out, float *out, cudaStream_t s) {
    const int64_t total = n_out * (w.k / Fmt<TYPE>::VPB);
    if (total == 0) return 0;
    const int threads = 128;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 64) blocks = 148 * 64;
    dequant_rows_kernel<TYPE><<<(unsigned)blocks, threads, 0, s>>>(w.tiles, w.n, w.k, w.kt, idx, n_out, out, w.status);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, "dequantize launch");
}

static int dequant_dispatch(const Weight &w, const int32_t *idx, int64_t n_out, float *out, cudaStream_t s) {
    switch (w.type) {
    case kQ4_0: return dequant_t<kQ4_0>(w, idx, n_out, out, s);
    case kQ8_0: return dequant_t<kQ8_0>(w, idx, n_out, out, s);
    case kQ4_K: return dequant_t<kQ4_K>(w, idx, n_out, out, s);
    case kQ6_K: return dequant_t<kQ6_K>(w, idx, n_out, out, s);
    }
    return fail(B200Q_ENOTIMPL, "dequantize: unsupported GGML type");
}

int launch_dequantize(const Weight &w, float *out, cudaStream_t s) { return dequant_dispatch(w, nullptr, w.n, out, s); }

int launch_gather(const Weight &w, const int32_t *idx, int64_t n_idx, float *out, cudaStream_t s) {
    return dequant_dispatch(w, idx, n_idx, out, s);
}

}  // namespace b200q
