// extern "C" entry points of libta_b200.so (declared in include/ta_b200.h):
// argument checking, kernel selection, launch shapes, and the two small helper
// kernels (per-image grayscale mean, inverse affine matrices).
#include <cuda.h>
#include <cuda_runtime.h>
#include <limits.h>
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/ta_b200.h"
#include "ta_tables.cuh"

namespace ta {

// ----------------------------------------------------------------------------- errors
static thread_local char g_err[512] = "";

static int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static int cuda_fail(cudaError_t e, const char *what)
{
    return fail(TA_B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// ----------------------------------------------------------------------------- per-device state
constexpr int kMaxDevices = 16;
// crop/flip, nearest, bilinear, crop/flip 128-bit, crop/flip staged, bilinear mixed, mean pre-pass, two-phase x 3;
// then nearest, bilinear, crop/flip staged, bilinear mixed on short tiles
constexpr int kNumKinds = 14, kNumDtypes = 4;
// TA_B200_SCALAR_DIRECT=1 keeps crop/flip launches on the 32-bit kernel (tests compare the two).
static const bool g_force_scalar_direct = [] { const char *e = getenv("TA_B200_SCALAR_DIRECT"); return e && e[0] == '1'; }();
// Which kernel runs a call without a matrix: 0 = choose by size, 1 = always the crop kernels,
// 2 = the staged kernel whenever the tensors allow it (ta_b200_debug_crop_path).
static std::atomic<int> g_crop_path{0};
// Tile height of the staged kernel for float images: 0 = by output height (ta_b200_debug_tile_height).
static std::atomic<int> g_tile_height{0};
// Limit of the kernels' barrier waits, and (diagnostics) the tile whose producer withholds its
// arrival in launches of the staged kernel: ta_b200_debug_wait().
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;
static std::atomic<unsigned long long> g_wait_ns{kDefaultWaitNs};
static std::atomic<int> g_skip_arrive_tile{-1};
// ta_b200_fused_augment_mean(): 0 = the two-launch sequence (default), 1 / 2 = one cooperative launch
// where possible, with the fused pass one / two images behind the reduction (ta_b200_mean_path)
static std::atomic<int> g_two_phase{0};

struct DeviceState {
    std::mutex mu;
    bool probed = false;
    int sm_count = 0;
    int cc_major = 0;
    unsigned long long *counters = nullptr;          // 4 words of device memory
    unsigned *status = nullptr;                      // pinned, mapped host word the kernels set on a time-out
    // launch shape per kernel: resident CTAs per SM (0 = not prepared yet)
    unsigned char blocks_per_sm[kNumKinds][kNumDtypes][2][kNumFlagCombos + 1] = {};
};
static DeviceState g_dev[kMaxDevices];

static int current_device(DeviceState **out, int *index)
{
    int d = -1;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (d < 0 || d >= kMaxDevices) return fail(TA_B200_ERR_DEVICE, "device index %d not supported", d);
    DeviceState &s = g_dev[d];
    std::lock_guard<std::mutex> lock(s.mu);
    if (!s.probed) {
        cudaDeviceProp prop;
        e = cudaGetDeviceProperties(&prop, d);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
        s.sm_count = prop.multiProcessorCount;
        s.cc_major = prop.major;
        if (prop.major != 10)
            return fail(TA_B200_ERR_DEVICE, "device %d is compute capability %d.%d; this library is built for 10.x only",
                        d, prop.major, prop.minor);
        e = cudaMalloc(&s.counters, 4 * sizeof(unsigned long long));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(counters)");
        e = cudaMemset(s.counters, 0, 4 * sizeof(unsigned long long));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(counters)");
        e = cudaHostAlloc((void **)&s.status, 64, cudaHostAllocMapped | cudaHostAllocPortable);
        if (e != cudaSuccess) return cuda_fail(e, "cudaHostAlloc(status word)");
        *s.status = 0u;
        s.probed = true;
    }
    *out = &s;
    if (index) *index = d;
    return TA_B200_OK;
}

// A barrier wait of an earlier launch on this device ran out: that launch left part of its output
// unwritten.  Read from the host-mapped word, so no synchronisation; stays raised until
// ta_b200_status(1) acknowledges it.
static int pending_timeout(const DeviceState &s)
{
    if (s.status && *(volatile unsigned *)s.status != 0u)
        return fail(TA_B200_ERR_TIMEOUT, "a barrier wait of an earlier launch on this device ran out and that launch left "
                    "its output incomplete; acknowledge with ta_b200_status(1)");
    return TA_B200_OK;
}

// bytes per element of `in` / of `out` and the factor vectors
static size_t in_bytes(int dtype) { return dtype == TA_B200_F32 ? 4 : dtype == TA_B200_F16 ? 2 : 1; }
static size_t out_bytes(int dtype) { return dtype == TA_B200_F16 || dtype == TA_B200_U8_F16 ? 2 : 4; }

static const KernelTable &table_for(int kind, int dtype, bool short_tiles)
{
    if (short_tiles)              // float and half images only (launch_fused)
        return dtype == TA_B200_F16 ? (kind == 1 ? table_f16_short_nearest() : table_f16_short_bilinear())
               : kind == 1 ? table_f32_short_nearest() : kind == 2 ? table_f32_short_bilinear()
               : kind == 3 ? table_f32_short_crop_staged() : table_f32_short_bilinear_mix();
    if (dtype == TA_B200_U8)      // staged kernels only (launch_fused never asks for kind 0)
        return kind == 1 ? table_u8_nearest() : kind == 2 ? table_u8_bilinear() : kind == 3 ? table_u8_crop_staged()
                                                                                           : table_u8_bilinear_mix();
    if (dtype == TA_B200_U8_F16)
        return kind == 1 ? table_u8h_nearest() : kind == 2 ? table_u8h_bilinear() : table_u8h_crop_staged();
    if (dtype == TA_B200_F32)
        return kind == 0 ? table_f32_direct() : kind == 1 ? table_f32_nearest() : kind == 2 ? table_f32_bilinear()
               : kind == 3 ? table_f32_crop_staged() : table_f32_bilinear_mix();
    return kind == 0 ? table_f16_direct() : kind == 1 ? table_f16_nearest() : table_f16_bilinear();
}

// Resident CTAs per SM for a kernel, computed once per device; also opts the kernel in
// to its dynamic shared memory size on that device.
static int prepare_kernel(DeviceState &s, const KernelEntry &ke, int kind, int dtype, int c, unsigned slot, int *blocks)
{
    std::lock_guard<std::mutex> lock(s.mu);
    unsigned char &cached = s.blocks_per_sm[kind][dtype][c == 3][slot];
    if (cached == 0) {
        const size_t smem = ke.smem;
        const void *fn = ke.fn;
        cudaError_t e;
        if (smem > 0) {
            e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(shared memory)");
        }
        int nb = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, fn, ke.threads, smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
        if (nb < 1) return fail(TA_B200_ERR_CUDA, "kernel does not fit on an SM");
        cached = (unsigned char)(nb > 255 ? 255 : nb);
    }
    *blocks = cached;
    return TA_B200_OK;
}

// ----------------------------------------------------------------------------- parameter block
// The caller's block in the current layout.  Two layouts are accepted: the current one and the
// one that ended before fill_rgb (its extra fields read as zero).  Any other struct_size is kept
// as it is, for validate() to refuse.
struct Imported {
    ta_b200_fused_params full;
    const ta_b200_fused_params *ptr;
    explicit Imported(const ta_b200_fused_params *p) : ptr(p)
    {
        if (p && p->struct_size == offsetof(ta_b200_fused_params, fill_rgb)) {
            memset(&full, 0, sizeof(full));
            memcpy(&full, p, offsetof(ta_b200_fused_params, fill_rgb));
            full.struct_size = sizeof(full);
            ptr = &full;
        }
    }
};

// ----------------------------------------------------------------------------- validation
static int validate(const ta_b200_fused_params *p, bool for_mean = false)
{
    if (!p) return fail(TA_B200_ERR_NULL, "params is NULL");
    if (p->struct_size != sizeof(ta_b200_fused_params))
        return fail(TA_B200_ERR_SHAPE, "struct_size %u is neither %zu nor %zu (ABI mismatch)", p->struct_size,
                    sizeof(ta_b200_fused_params), offsetof(ta_b200_fused_params, fill_rgb));
    if (p->dtype != TA_B200_F32 && p->dtype != TA_B200_F16 && p->dtype != TA_B200_U8 && p->dtype != TA_B200_U8_F16)
        return fail(TA_B200_ERR_DTYPE, "dtype %d", p->dtype);
    if (p->c != 1 && p->c != 3)
        return fail(TA_B200_ERR_SHAPE, "channels must be 1 or 3, got %d", p->c);
    if (p->n < 0 || p->h <= 0 || p->w <= 0 || p->oh <= 0 || p->ow <= 0)
        return fail(TA_B200_ERR_SHAPE, "bad sizes n=%d h=%d w=%d oh=%d ow=%d", p->n, p->h, p->w, p->oh, p->ow);
    if ((double)p->h * p->w >= 2147483648.0 || (double)p->oh * p->ow >= 2147483648.0)
        return fail(TA_B200_ERR_TOO_LARGE, "one image plane must stay below 2^31 elements");
    // (the grayscale-mean pre-pass writes no image: it needs `in` only)
    if (p->n > 0 && (!p->in || (!p->out && !for_mean))) return fail(TA_B200_ERR_NULL, "in/out is NULL");
    if (p->c == 1 && (p->apply & (TA_B200_APPLY_SATURATION | TA_B200_APPLY_GRAYSCALE)))
        return fail(TA_B200_ERR_UNSUPPORTED, "saturation / grayscale need 3 channels");
    if ((p->apply & TA_B200_APPLY_BRIGHTNESS) && !p->brightness) return fail(TA_B200_ERR_NULL, "brightness is NULL");
    if (p->matrix && p->interp != TA_B200_NEAREST && p->interp != TA_B200_BILINEAR)
        return fail(TA_B200_ERR_UNSUPPORTED, "interp %d", p->interp);
    if (p->dtype == TA_B200_U8_F16 && (for_mean || ((p->apply & TA_B200_APPLY_CONTRAST) && p->contrast_mode == TA_B200_CONTRAST_MEAN)))
        return fail(TA_B200_ERR_UNSUPPORTED, "the grayscale-mean contrast reads bytes into float32 pixels only");
    if (for_mean) return TA_B200_OK;     // the pre-pass reads geometry and brightness only
    if ((p->apply & TA_B200_APPLY_CONTRAST) && !p->contrast) return fail(TA_B200_ERR_NULL, "contrast is NULL");
    if ((p->apply & TA_B200_APPLY_SATURATION) && !p->saturation) return fail(TA_B200_ERR_NULL, "saturation is NULL");
    if ((p->apply & TA_B200_APPLY_GRAYSCALE) && !p->gray) return fail(TA_B200_ERR_NULL, "gray is NULL");
    if (p->apply & ~31u) return fail(TA_B200_ERR_UNSUPPORTED, "unknown apply bits 0x%x", p->apply);
    if (p->contrast_mode != TA_B200_CONTRAST_FAST && p->contrast_mode != TA_B200_CONTRAST_MEAN)
        return fail(TA_B200_ERR_UNSUPPORTED, "contrast_mode %d", p->contrast_mode);
    if ((p->apply & TA_B200_APPLY_CONTRAST) && p->contrast_mode == TA_B200_CONTRAST_MEAN && !p->gray_mean)
        return fail(TA_B200_ERR_NULL, "contrast_mode MEAN needs gray_mean");
    return TA_B200_OK;
}

static int validate_geometry_only(const ta_b200_fused_params *p) { return validate(p, true); }

// How many of a reference thread's 8 pixels get the other x contraction, per colour-flag
// combination (late_x() in ta_common.cuh; measured against the reference's kernels on a
// B200, fp32, bilinear, neither output dimension divisible by 16; 0 elsewhere).
static int late_count_of(const ta_b200_fused_params *p)
{
    static const unsigned char late_count[32] = {0, 0, 0, 0, 0, 1, 1, 3, 0, 2, 1, 3, 0, 2, 2, 3,
                                                 0, 0, 0, 0, 0, 1, 2, 3, 0, 2, 1, 3, 0, 2, 2, 3};
    if (p->matrix && p->interp == TA_B200_BILINEAR && out_bytes(p->dtype) == 4 && p->oh % 16 != 0 && p->ow % 16 != 0)
        return late_count[p->apply & 31u];
    return 0;
}

static void fill_kargs(KArgs &k, const ta_b200_fused_params *p, DeviceState &s)
{
    memset(&k, 0, sizeof(k));
    k.in = p->in; k.out = p->out;
    k.top = p->top; k.left = p->left; k.flip = p->flip; k.matrix = p->matrix;
    k.bf = p->brightness; k.cf = p->contrast; k.sf = p->saturation; k.gray = p->gray;
    k.gray_mean = p->gray_mean;
    k.counters = s.counters;
    k.status = s.status;
    k.wait_ns = g_wait_ns.load(std::memory_order_relaxed);
    k.skip_arrive_tile = g_skip_arrive_tile.load(std::memory_order_relaxed);
    k.n = p->n; k.h = p->h; k.w = p->w; k.oh = p->oh; k.ow = p->ow;
    for (int i = 0; i < 3; ++i) k.fill[i] = p->fill_per_channel ? p->fill_rgb[i] : p->fill;
    for (int i = 0; i < 3; ++i) {
        const bool norm = (p->apply & TA_B200_APPLY_NORMALIZE) != 0;
        k.mean[i] = norm ? p->mean[i] : 0.0f;
        k.stdv[i] = norm ? p->std[i] : 1.0f;
        k.inv_std[i] = 1.0f / k.stdv[i];
        k.nbias[i] = -k.mean[i] * k.inv_std[i];
    }
    k.late_x_slot = 8 - late_count_of(p);
    k.pair_store = out_bytes(p->dtype) == 2 && p->ow % 2 == 0 && ((uintptr_t)p->out % 4) == 0;
    const size_t es = in_bytes(p->dtype);
    k.staged_ok = ((size_t)p->w * es) % 16 == 0 && ((uintptr_t)p->in % 16) == 0 &&
                  ((size_t)p->h * p->w * es) % 16 == 0 &&
                  // the staged path converts coordinates with a 2^22-range shortcut
                  p->h < (1 << 22) && p->w < (1 << 22) && p->oh < (1 << 22) && p->ow < (1 << 22);
}

static unsigned template_flags(const ta_b200_fused_params *p)
{
    unsigned f = p->apply & 31u;
    if ((f & kC) && p->contrast_mode == TA_B200_CONTRAST_MEAN) f |= kMean;
    return f;
}

// cuTensorMapEncodeTiled, fetched through the runtime so the library does not link libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return (EncodeTiledFn)sym;
    }();
    return fn;
}

// Tensor maps over the input seen as [n*c, h, w]: boxes of pitch_of(element size) columns x 8, 16,
// ... kMaxRows rows x 1 plane, out-of-range elements read as zero.
static int build_tensor_maps(TMaps &maps, const ta_b200_fused_params *p)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(TA_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const size_t es = in_bytes(p->dtype);
    const CUtensorMapDataType dt = es == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : es == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const cuuint64_t dims[3] = {(cuuint64_t)p->w, (cuuint64_t)p->h, (cuuint64_t)p->n * p->c};
    const cuuint64_t strides[2] = {(cuuint64_t)p->w * es, (cuuint64_t)p->w * p->h * es};
    const cuuint32_t estr[3] = {1, 1, 1};
    for (int g = 0; g < kNumGroups; ++g) {
        const cuuint32_t box[3] = {(cuuint32_t)pitch_of((int)es), (cuuint32_t)((g + 1) * kGroupRows), 1};
        CUresult r = enc(&maps.rows[g], dt,
                         3, const_cast<void *>(p->in), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(TA_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    }
    return TA_B200_OK;
}

// first_image: index of p's first image in the batch the caller is working through in pieces (the
// host-buffer pipeline); the per-pixel rule of late_x() follows the index within that batch, as one
// launch of the reference over the whole batch would.
static int launch_fused(const ta_b200_fused_params *p, cudaStream_t stream, bool checked, unsigned first_image = 0)
{
    int rc = validate(p);
    if (rc != TA_B200_OK) return rc;
    if (p->n == 0) return TA_B200_OK;
    DeviceState *s = nullptr;
    rc = current_device(&s, nullptr);
    if (rc != TA_B200_OK) return rc;
    rc = pending_timeout(*s);
    if (rc != TA_B200_OK) return rc;

    KArgs k;
    fill_kargs(k, p, *s);
    k.lin_base = first_image * (unsigned)p->oh * (unsigned)p->ow;      // modulo 2^32: late_x() reads bits 7-9
    int kind = p->matrix ? (p->interp == TA_B200_BILINEAR ? 2 : 1) : 0;
    if (kind == 0 && p->dtype == TA_B200_F32 && k.staged_ok) {
        // Large fp32 batches run faster through the staged kernel (tensor copies cost no
        // instructions): measured 264 us instead of 288 us on 64 x 3 x 1280^2 -> 1024^2 with all
        // colour operations, bit-identical output.  Small or narrow outputs and fp16 do not gain.
        const int path = g_crop_path.load(std::memory_order_relaxed);
        const bool large = p->ow >= 160 && (double)p->n * p->c * p->oh * p->ow * 4.0 >= 32.0 * 1024 * 1024;
        if (path == 2 || (path == 0 && large)) {
            kind = 3;
            k.fill[0] = k.fill[1] = k.fill[2] = 0.0f;
        }
    }
    if (kind == 0 && in_bytes(p->dtype) == 1) {     // bytes are read by the staged kernels only
        kind = 3;
        k.fill[0] = k.fill[1] = k.fill[2] = 0.0f;
    }
    unsigned f = template_flags(p);
    if (kind == 2 && k.late_x_slot < 8 && !checked) kind = 4;     // only swapped fp32 variants get here (fill_kargs)
    // Small outputs whose height leaves the last row of 64-row tiles at most half full run on 64 x 32
    // tiles with a deeper ring: with few tiles per image the number of tiles in flight matters more
    // than the pixels per thread (ta_affine.cuh).  Measured limits: float images up to 256 output
    // rows (224: 224 against 236 us per 1024 images; 288: 369 against 357), half images up to 96
    // (96: 164 / 222 against 169 / 250 us per 4096 images; 224: 189 against 167).  Float images
    // without a matrix always do: their consumers have so little to do per pixel that the ring is
    // what matters (160 x 3 x 704^2 -> 640^2: 252 against 290 us on two GPUs; 80 x 3 x 1024^2 -> 896^2:
    // 246 against 283 us on one GPU, 252 against 246 us on another; 64 x 3 x 1280^2 -> 1024^2: 261
    // against 258 us: never more than 2.5 % behind, up to 15 % ahead).  Same arithmetic per pixel,
    // hence the same output.
    const int last_rows = p->oh % kTileH, forced = g_tile_height.load(std::memory_order_relaxed);
    const bool has_short = p->dtype == TA_B200_F32 || p->dtype == TA_B200_F16;
    const bool small = last_rows != 0 && last_rows <= kTileHShort && p->oh <= (p->dtype == TA_B200_F32 ? 256 : 96);
    const bool short_tiles = kind != 0 && has_short &&
                             (forced ? forced == kTileHShort : small || (kind == 3 && p->dtype == TA_B200_F32));
    const int tile_h = short_tiles ? kTileHShort : kTileH;
    const KernelTable &tab = table_for(kind, p->dtype, short_tiles);
    unsigned slot = f;
    const KernelEntry *ke;
    if (checked && kind != 0) {
        if (f != 0) return fail(TA_B200_ERR_UNSUPPORTED, "checked staging build exists for apply == 0 only");
        ke = p->c == 3 ? &tab.c3_checked : &tab.c1_checked;
        slot = kNumFlagCombos;
    } else {
        ke = p->c == 3 ? &tab.c3[f] : &tab.c1[f];
    }
    // Crop/flip only: the 128-bit kernel needs whole-vector output rows and vector-aligned tensors.
    const size_t es_bytes = in_bytes(p->dtype);
    const int epv = (int)(16 / es_bytes);
    // (every channel plane a whole number of vectors: the kernel takes the shift of a strip from
    // its first channel)
    const bool vec = kind == 0 && !g_force_scalar_direct && p->ow % epv == 0 && ((uintptr_t)p->in % 16) == 0 &&
                     ((uintptr_t)p->out % 16) == 0 && ((size_t)p->h * p->w * es_bytes) % 16 == 0;
    if (vec) ke = p->c == 3 ? &tab.c3_vec[f] : &tab.c1_vec[f];
    if (!ke->fn) return fail(TA_B200_ERR_UNSUPPORTED, "no kernel for channels=%d flags=0x%x", p->c, f);
    int blocks = 0;
    const int kind_index = short_tiles ? 9 + kind : vec ? 3 : kind == 3 ? 4 : kind == 4 ? 5 : kind;       // short: 10 .. 13
    rc = prepare_kernel(*s, *ke, kind_index, p->dtype, p->c, slot, &blocks);
    if (rc != TA_B200_OK) return rc;

    long long work;
    if (vec) {
        k.tiles_x = (p->ow + 32 * epv - 1) / (32 * epv);
        k.tiles_y = (p->oh + kVecRows - 1) / kVecRows;
        work = ((long long)p->n * k.tiles_x * k.tiles_y + kWarps - 1) / kWarps;
    } else if (kind == 0) {
        k.tiles_x = (p->ow + 31) / 32;
        k.tiles_y = (p->oh + kDirectRows - 1) / kDirectRows;
        work = ((long long)p->n * k.tiles_x * k.tiles_y + kWarps - 1) / kWarps;      // CTAs needed at one strip per warp
    } else {
        k.tiles_x = (p->ow + kTileW - 1) / kTileW;
        k.tiles_y = (p->oh + tile_h - 1) / tile_h;
        work = (long long)p->n * k.tiles_x * k.tiles_y;
    }
    const long long tiles = (long long)p->n * k.tiles_x * k.tiles_y;
    // 32-bit tile counters in the kernels are stepped past the end by up to a few grid strides
    if (tiles >= 2147483647LL - (1 << 24)) return fail(TA_B200_ERR_TOO_LARGE, "too many tiles (%lld)", tiles);
    k.num_tiles = (int)tiles;
    // Persistent launch: one wave of resident CTAs, fewer when there is less work.
    long long grid = (long long)s->sm_count * blocks;
    if (grid > work) grid = work;
    if (grid < 1) grid = 1;
    cudaError_t e;
    if (kind == 0) {
        void *args[] = {&k};
        e = cudaLaunchKernel(ke->fn, dim3((unsigned)grid), dim3(ke->threads), args, ke->smem, stream);
    } else {
        TMaps maps;
        memset(&maps, 0, sizeof(maps));
        if (k.staged_ok) {
            // dimensions beyond what a tensor map can describe: gather everything directly
            if ((double)p->n * p->c >= 2147483648.0) k.staged_ok = 0;
            else {
                rc = build_tensor_maps(maps, p);
                if (rc != TA_B200_OK) return rc;
            }
        }
        void *args[] = {&k, &maps};
        e = cudaLaunchKernel(ke->fn, dim3((unsigned)grid), dim3(ke->threads), args, ke->smem, stream);
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernel(fused)");
    return TA_B200_OK;
}

}  // namespace ta

#include "ta_api_helpers.cuh"

// ----------------------------------------------------------------------------- allocation-free pre-pass
// ta_b200_gray_mean_static(): the grayscale-mean pre-pass for callers that may not allocate.
// Its scratch is this fixed array in device memory.  Every GPU that loads the library carries
// the array until the process exits, and every call on a device uses the same bytes.
namespace ta {

constexpr size_t kStaticScratchBytes = 1u << 20;                       // 1 MiB per device
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address;
// the address a kernel can use is looked up once per device, with that device current.
static std::mutex g_static_mu;
static void *g_static_ptr[kMaxDevices] = {};

static int static_scratch_for_current_device(void **out)
{
    int d = -1;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (d < 0 || d >= kMaxDevices) return fail(TA_B200_ERR_DEVICE, "device index %d not supported", d);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[d]) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        if (major != 10) return fail(TA_B200_ERR_DEVICE, "device %d is not compute capability 10.x", d);
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        if (!ptr) return fail(TA_B200_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_static_ptr[d] = ptr;
    }
    *out = g_static_ptr[d];
    return TA_B200_OK;
}

static int gray_mean_static(const ta_b200_fused_params *p, float *mean_out, cudaStream_t stream)
{
    int rc = validate_geometry_only(p);
    if (rc != TA_B200_OK) return rc;
    if (!mean_out) return fail(TA_B200_ERR_NULL, "mean_out is NULL");
    if (p->n == 0) return TA_B200_OK;
    if (p->n > 65535) return fail(TA_B200_ERR_TOO_LARGE, "at most 65535 images per call");
    if (in_bytes(p->dtype) == 1) return fail(TA_B200_ERR_UNSUPPORTED, "the built-in scratch serves float images only");
    const int bpi = mean_blocks_per_image(p->oh, p->ow);
    const size_t need = mean_partials_offset(p->n) + (size_t)p->n * bpi * sizeof(float);
    if (need > kStaticScratchBytes)
        return fail(TA_B200_ERR_TOO_LARGE,
                    "this call needs %zu bytes of scratch but the built-in buffer holds %zu: pass fewer images per call "
                    "(%d images of %dx%d need %d partial sums each) or use ta_b200_gray_mean with your own scratch",
                    need, kStaticScratchBytes, p->n, p->oh, p->ow, bpi);
    void *scratch = nullptr;
    rc = static_scratch_for_current_device(&scratch);
    if (rc != TA_B200_OK) return rc;
    static DeviceState no_counters;                                    // only its null `counters` and `status` are read
    KArgs k;
    fill_kargs(k, p, no_counters);
    unsigned *counters = (unsigned *)scratch;
    float *partials = (float *)((char *)scratch + mean_partials_offset(p->n));
    // The tickets must start at zero; the previous call (possibly with another n) left its own there.
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)p->n * sizeof(unsigned), stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(static scratch)");
    const int kind = p->matrix ? (p->interp == TA_B200_BILINEAR ? 2 : 1) : 0;
    const bool bright = (p->apply & TA_B200_APPLY_BRIGHTNESS) != 0;
    e = p->dtype == TA_B200_F32
            ? launch_gray_mean<float>(k, p->c, kind, bright, mean_out, counters, partials, bpi, stream)
            : launch_gray_mean<__half>(k, p->c, kind, bright, mean_out, counters, partials, bpi, stream);
    if (e != cudaSuccess) return cuda_fail(e, "launch(gray_mean, static scratch)");
    return TA_B200_OK;
}

}  // namespace ta

extern "C" int ta_b200_gray_mean_static(const ta_b200_fused_params *p, float *mean_out, void *stream)
{
    return ta::gray_mean_static(ta::Imported(p).ptr, mean_out, (cudaStream_t)stream);
}
