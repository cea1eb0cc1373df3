// Checkpoint layouts -> the layout the product kernels read: one AWQ or GPTQ layer
// (`qweight`, `qzeros`, `scales`) as MLX's affine codes, scales and biases
// (convert_packed, crates/nuvec-lm/src/quant.rs:36-199), on the device, so a loader uploads the
// file's bytes as they are and converts them in place of the reference's host loops.
//
//   codes   AWQ   qweight int32 [inputs, outputs / 8]: value c of eight neighbouring outputs sits in
//                 nibble AWQ_ORDER[c] = {0, 4, 1, 5, 2, 6, 3, 7}[c] of the word (4-bit only);
//           GPTQ  qweight int32 [inputs * bits / 32, outputs]: a word holds 32 / bits consecutive
//                 inputs of one output, low bits first -- MLX's packing along the inputs already, so
//                 the conversion is the transpose of a matrix of 32-bit words;
//           out   uint32 [outputs, inputs * bits / 32], input i of a row at bits (i % per_word) * bits
//                 of word i / per_word;
//   zeros   qzeros int32 [groups, outputs * bits / 32] packed like the codes of its format along the
//           outputs (GPTQ v1 stores zero - 1); absent: 2^(bits - 1);
//   scales  [groups, outputs] -> [outputs, groups], unchanged bits;
//   biases  -zero (float32) times the scale (float32), rounded to the scales' type, [outputs, groups].
//
// gpt-oss's MXFP4 `*_blocks` need no kernel: their bytes are MLX's codes already (quant.rs:24-34) and the
// gate / up rows are taken apart with nvc_take_strided (below).
#include "common.cuh"

namespace nvc {

__device__ __constant__ int kAwqOrder[8] = {0, 4, 1, 5, 2, 6, 3, 7};

// AWQ codes.  A block turns a tile of 64 inputs x 256 outputs (64 rows x 32 words of qweight) into
// 256 rows x 8 words of the result through shared memory: 128-byte reads, 32-byte writes.
__global__ void __launch_bounds__(256) awq_codes_kernel(const uint32_t *__restrict__ words, uint32_t *__restrict__ out, int64_t inputs, int64_t cols) {
    __shared__ uint32_t tile[64][33];
    const int t = threadIdx.x;
    const int64_t i0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 32, W = inputs / 8;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int r = j * 8 + (t >> 5), c = t & 31;
        tile[r][c] = (i0 + r < inputs && c0 + c < cols) ? words[(i0 + r) * cols + c0 + c] : 0u;
    }
    __syncthreads();
    const int oc = t >> 3, c = t & 7;  // output c0 * 8 + t
    if (c0 + oc >= cols) return;
    const int shift = 4 * kAwqOrder[c];
    uint32_t *dst = out + ((c0 + oc) * 8 + c) * W + i0 / 8;
    uint32_t made[8];
#pragma unroll
    for (int wi = 0; wi < 8; wi++) {
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) word |= ((tile[wi * 8 + k][oc] >> shift) & 15u) << (4 * k);
        made[wi] = word;
    }
    if (i0 + 64 <= inputs && ((uintptr_t)dst & 15) == 0) {  // the thread's 32 bytes as two 16-byte stores
        reinterpret_cast<uint4 *>(dst)[0] = make_uint4(made[0], made[1], made[2], made[3]);
        reinterpret_cast<uint4 *>(dst)[1] = make_uint4(made[4], made[5], made[6], made[7]);
    } else {
#pragma unroll
        for (int wi = 0; wi < 8; wi++)
            if (i0 + wi * 8 < inputs) dst[wi] = made[wi];
    }
}

// out[o, j, :] = src[o, first + j * step, :] for rows of inner_bytes bytes, in units of UNIT bytes.
template <typename U>
__global__ void __launch_bounds__(256) take_strided_kernel(const U *__restrict__ src, U *__restrict__ out, int64_t n, int64_t picked, int64_t inner,
                                                           int64_t first, int64_t step, int64_t total) {
    for (int64_t at = (int64_t)blockIdx.x * 256 + threadIdx.x; at < total; at += (int64_t)gridDim.x * 256) {
        const int64_t c = at % inner, row = at / inner;
        const int64_t j = row % picked, o = row / picked;
        out[at] = src[(o * n + first + j * step) * inner + c];
    }
}

// GPTQ codes: out[o][w] = words[w][o], 32 x 32 tiles through shared memory.
__global__ void __launch_bounds__(256) transpose_words_kernel(const uint32_t *__restrict__ words, uint32_t *__restrict__ out, int64_t rows, int64_t cols) {
    __shared__ uint32_t tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int r = ty + 8 * j;
        if (r0 + r < rows && c0 + tx < cols) tile[r][tx] = words[(r0 + r) * cols + c0 + tx];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int c = ty + 8 * j;
        if (c0 + c < cols && r0 + tx < rows) out[(c0 + c) * rows + r0 + tx] = tile[tx][c];
    }
}

// scales [groups, outputs] -> [outputs, groups]; biases = -zero * scale.
template <typename T>
__global__ void __launch_bounds__(256) packed_scales_kernel(const T *__restrict__ scales, const uint32_t *__restrict__ qzeros, T *__restrict__ out_scales,
                                                            T *__restrict__ out_biases, int64_t groups, int64_t outputs, int format, int bits) {
    const int64_t at = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // g * outputs + o: reads along the outputs
    if (at >= groups * outputs) return;
    const int64_t g = at / outputs, o = at % outputs;
    const int per_word = 32 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    float zero;
    if (qzeros == nullptr) {
        zero = (float)(1u << (bits - 1));
    } else {
        const int64_t zc = (outputs + per_word - 1) / per_word;
        const uint32_t w = qzeros[g * zc + o / per_word];
        const int shift = format == 0 ? 4 * kAwqOrder[o % per_word] : bits * (int)(o % per_word);
        zero = (float)(((w >> shift) & mask) + (format == 1 ? 1u : 0u));
    }
    const T s = scales[at];
    out_scales[o * groups + g] = s;
    DT<T>::store(out_biases, (size_t)(o * groups + g), __fmul_rn(-zero, DT<T>::load(&s, 0)));
}

}  // namespace nvc

using namespace nvc;

extern "C" int32_t nvc_convert_packed(nvc_device *dev, int32_t format, int32_t bits, int32_t group_size, int32_t scale_dtype, const int32_t *qweight,
                                      const int32_t *qzeros, const void *scales, int64_t inputs, int64_t outputs, uint32_t *out_codes,
                                      void *out_scales, void *out_biases) {
    NVC_TRY(make_current(dev));
    if (format < NVC_PACKED_AWQ || format > NVC_PACKED_GPTQ_V2) return set_error(NVC_ERR_INVALID_ARGUMENT, "convert_packed: unknown format %d", format);
    if (bits != 2 && bits != 4 && bits != 8) return set_error(NVC_ERR_UNSUPPORTED, "convert_packed: %d-bit codes (2, 4 or 8 fill a word)", bits);
    if (format == NVC_PACKED_AWQ && bits != 4) return set_error(NVC_ERR_UNSUPPORTED, "convert_packed: AWQ packs 4-bit codes, got %d bits", bits);
    if (group_size <= 0 || inputs < 0 || outputs < 0) return set_error(NVC_ERR_INVALID_ARGUMENT, "convert_packed: invalid shape");
    const int per_word = 32 / bits;
    if (inputs % group_size != 0 || inputs % per_word != 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "convert_packed: %lld inputs do not match groups of %d", (long long)inputs, group_size);
    if (format == NVC_PACKED_AWQ && outputs % per_word != 0)
        return set_error(NVC_ERR_INVALID_ARGUMENT, "convert_packed: %lld outputs are not whole words of %d", (long long)outputs, per_word);
    if (scale_dtype != NVC_F16 && scale_dtype != NVC_BF16 && scale_dtype != NVC_F32)
        return set_error(NVC_ERR_UNSUPPORTED, "convert_packed: scales of dtype %d", scale_dtype);
    if (inputs == 0 || outputs == 0) return NVC_OK;
    if (!qweight || !scales || !out_codes || !out_scales || !out_biases) return set_error(NVC_ERR_INVALID_ARGUMENT, "convert_packed: null operand");
    const int64_t groups = inputs / group_size;
    if (format == NVC_PACKED_AWQ) {
        const int64_t cols = outputs / 8;
        dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((inputs + 63) / 64));
        awq_codes_kernel<<<grid, 256, 0, dev->stream>>>((const uint32_t *)qweight, out_codes, inputs, cols);
        NVC_TRY(check_launch(dev, "awq_codes_kernel"));
    } else {
        const int64_t rows = inputs / per_word;
        dim3 grid((unsigned)((outputs + 31) / 32), (unsigned)((rows + 31) / 32));
        transpose_words_kernel<<<grid, 256, 0, dev->stream>>>((const uint32_t *)qweight, out_codes, rows, outputs);
        NVC_TRY(check_launch(dev, "transpose_words_kernel"));
    }
    const unsigned blocks = (unsigned)((groups * outputs + 255) / 256);
    if (scale_dtype == NVC_F16)
        packed_scales_kernel<__half><<<blocks, 256, 0, dev->stream>>>((const __half *)scales, (const uint32_t *)qzeros, (__half *)out_scales,
                                                                       (__half *)out_biases, groups, outputs, format, bits);
    else if (scale_dtype == NVC_BF16)
        packed_scales_kernel<__nv_bfloat16><<<blocks, 256, 0, dev->stream>>>((const __nv_bfloat16 *)scales, (const uint32_t *)qzeros,
                                                                              (__nv_bfloat16 *)out_scales, (__nv_bfloat16 *)out_biases, groups, outputs,
                                                                              format, bits);
    else
        packed_scales_kernel<float><<<blocks, 256, 0, dev->stream>>>((const float *)scales, (const uint32_t *)qzeros, (float *)out_scales,
                                                                     (float *)out_biases, groups, outputs, format, bits);
    return check_launch(dev, "packed_scales_kernel");
}

extern "C" int32_t nvc_take_strided(nvc_device *dev, const void *src, int64_t outer, int64_t n, int64_t inner_bytes, int64_t first, int64_t step,
                                    void *out) {
    NVC_TRY(make_current(dev));
    if (outer < 0 || n < 0 || inner_bytes < 0 || first < 0 || step < 1) return set_error(NVC_ERR_INVALID_ARGUMENT, "take_strided: invalid shape");
    const int64_t picked = first < n ? (n - first + step - 1) / step : 0;
    const int64_t bytes = outer * picked * inner_bytes;
    if (bytes == 0) return NVC_OK;
    if (!src || !out) return set_error(NVC_ERR_INVALID_ARGUMENT, "take_strided: null operand");
    const uintptr_t both = (uintptr_t)src | (uintptr_t)out | (uintptr_t)inner_bytes;
    const int unit = both % 16 == 0 ? 16 : both % 8 == 0 ? 8 : both % 4 == 0 ? 4 : both % 2 == 0 ? 2 : 1;
    const int64_t total = bytes / unit, inner = inner_bytes / unit;
    int64_t want = (total + 255) / 256, cap = (int64_t)dev->prop.multiProcessorCount * 16;
    const unsigned blocks = (unsigned)(want < cap ? want : cap);
    switch (unit) {
        case 16: take_strided_kernel<uint4><<<blocks, 256, 0, dev->stream>>>((const uint4 *)src, (uint4 *)out, n, picked, inner, first, step, total); break;
        case 8: take_strided_kernel<uint2><<<blocks, 256, 0, dev->stream>>>((const uint2 *)src, (uint2 *)out, n, picked, inner, first, step, total); break;
        case 4: take_strided_kernel<uint32_t><<<blocks, 256, 0, dev->stream>>>((const uint32_t *)src, (uint32_t *)out, n, picked, inner, first, step, total); break;
        case 2: take_strided_kernel<uint16_t><<<blocks, 256, 0, dev->stream>>>((const uint16_t *)src, (uint16_t *)out, n, picked, inner, first, step, total); break;
        default: take_strided_kernel<uint8_t><<<blocks, 256, 0, dev->stream>>>((const uint8_t *)src, (uint8_t *)out, n, picked, inner, first, step, total); break;
    }
    return check_launch(dev, "take_strided_kernel");
}
