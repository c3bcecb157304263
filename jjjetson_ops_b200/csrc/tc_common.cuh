// PTX wrappers shared by the tcgen05 GEMM kernels: tensor-memory loads and fences, the shared-memory
// matrix descriptor of the unswizzled K-major operand layout, and the stores that build such tiles.
#pragma once

#include <cuda.h>

#include "jq_common.cuh"

namespace jq {

// The driver's tensor-map encoder, looked up through the runtime so that the library does not link against libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn tensor_map_encoder() {
    static const EncodeTiledFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            f = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// Byte tensor [rows][row_len] with rows `pitch` bytes apart, copied in boxes of box_rows rows x box_bytes bytes
// (box_bytes a multiple of 16, at most 256; box_rows at most 256).  No swizzle: a box lands row after row.
inline int encode_byte_map(CUtensorMap *map, const void *base, uint64_t row_len, uint64_t rows, uint64_t pitch, uint32_t box_bytes,
                           uint32_t box_rows) {
    const EncodeTiledFn encode = tensor_map_encoder();
    if (encode == nullptr) return set_error(JQ_ERR_UNSUPPORTED, "the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {row_len, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t elem_strides[2] = {1u, 1u};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(JQ_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return JQ_OK;
}

}  // namespace jq

#ifdef __CUDACC__

namespace jq {

// One tiled tensor copy global -> shared: the box of `map` at byte column x, row y; completion counted in bytes on
// an mbarrier.  x must be a multiple of 16.  Rows past the end of the tensor arrive as zeros (and are counted).
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// One operand tile is 128 rows x 32 bytes (32 int8 or 16 fp16 values of K) in the tensor core's
// canonical K-major layout without swizzle: 8-row x 16-byte core matrices, the two 16-byte chunks of
// a row 128 bytes apart, groups of 8 rows 256 bytes apart.
constexpr int TC_TILE = 4096;
constexpr uint32_t TC_LBO = 128, TC_SBO = 256;

// position of the 16-byte K-chunk kc (0/1) of row r inside a tile
__device__ __forceinline__ uint32_t tile_off(int r, int kc) {
    return (uint32_t)((r >> 3) * TC_SBO + kc * TC_LBO + (r & 7) * 16);
}

// shared-memory matrix descriptor of a tile: K-major, no swizzle, version 1; `lbo` bytes between the 16-byte K-chunks
// of a row, `sbo` bytes between groups of 8 rows
__device__ __forceinline__ uint64_t tc_desc_strided(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) { return tc_desc_strided(smem_addr, TC_LBO, TC_SBO); }

__device__ __forceinline__ void sts_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 consecutive columns of 32-bit accumulator -> registers (completion: tcgen05.wait::ld)
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D(fp32, TMEM) (+)= A(fp16 tile) x B(fp16 tile)^T, K = 16
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

// All tensor-core operations this thread has issued so far arrive on the mbarrier when they complete.
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Instruction descriptor of kind::f16 with fp32 accumulation, fp16 A and B, both K-major:
// `rows_a` TMEM lanes (MMA M) by `rows_b` TMEM columns (MMA N).
__device__ __forceinline__ uint32_t tc_idesc_f16(int rows_a, int rows_b) {
    return (1u << 4) | ((uint32_t)(rows_b >> 3) << 17) | ((uint32_t)(rows_a >> 4) << 24);
}

}  // namespace jq

#endif  // __CUDACC__
