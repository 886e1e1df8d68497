// Second half of ta_api.cu: the two helper kernels and the extern "C" functions.
#pragma once

namespace ta {

// ----------------------------------------------------------------------------- grayscale mean
// Mean over the output window of gray(clamp(brightness * sample)), i.e. of the image that
// torchvision-exact contrast blends towards (triton_augment/functional.py:366-376 applied
// after geometry and brightness).  grid = (blocks per image, images).  Each block sums a
// fixed set of pixels in a fixed order, writes one partial, and the block that finishes
// last for an image adds that image's partials in index order, so the result does not
// depend on scheduling.  Nothing waits on anything.
constexpr int kMeanMaxBlocks = 128;

__host__ __device__ inline int mean_blocks_per_image(int oh, int ow)
{
    const long long px = (long long)oh * ow;
    long long b = (px + 4095) / 4096;
    return (int)(b < 1 ? 1 : b > kMeanMaxBlocks ? kMeanMaxBlocks : b);
}

// scratch layout: [n] unsigned counters, padded to 256 bytes, then [n][bpi] float partials
__host__ __device__ inline size_t mean_partials_offset(int n)
{
    return (((size_t)n * sizeof(unsigned)) + 255) / 256 * 256;
}

template <typename T, int C, int KIND, bool BRIGHT>
__global__ void __launch_bounds__(kThreads) gray_mean_kernel(const __grid_constant__ KArgs k, float *mean_out,
                                                              unsigned *counters, float *partials)
{
    const int n = blockIdx.y, blk = blockIdx.x, bpi = gridDim.x;
    Geom g;
    load_geom(g, k, n, KIND != 0);
    const T *img = (const T *)k.in + (size_t)n * C * k.h * k.w;
    const size_t plane = (size_t)k.h * k.w;
    T fillv[C];
#pragma unroll
    for (int c = 0; c < C; ++c) fillv[c] = Elem<T>::from_f(KIND != 0 ? k.fill[c] : 0.0f);
    float bf = 1.0f;
    __half bh = __float2half_rn(1.0f);
    if (BRIGHT) {
        if (sizeof(T) == 4) bf = ((const float *)k.bf)[n];
        else bh = ((const __half *)k.bf)[n];
    }
    const int total = k.oh * k.ow;
    float acc = 0.0f;
    for (int p = blk * kThreads + threadIdx.x; p < total; p += bpi * kThreads) {
        const int y = p / k.ow, x = p - y * k.ow;
        float v[C];
        if (KIND == 0) {
            const int xin = (int)img_x(g, k.ow, x), yin = (int)img_y(g, y);
#pragma unroll
            for (int c = 0; c < C; ++c) v[c] = Elem<T>::to_f(tap_global(img + c * plane, k.w, k.h, xin, yin, fillv[c]));
        } else {
            const float xc = centred(img_x(g, k.ow, x), g.half_w), yc = centred(img_y(g, y), g.half_h);
            // the common recipe of the sampling mode; the rarer swapped one moves a coordinate by
            // one ulp at most, which is invisible in a mean over the whole window
            const float sx = src_coord_r<CoordRecipe<KIND, 0u>::x>(xc, yc, g.a, g.b, g.c, g.half_w);
            const float sy = src_coord_r<CoordRecipe<KIND, 0u>::y>(xc, yc, g.d, g.e, g.f, g.half_h);
            if (KIND == 1) {
                const int xn = __float2int_rn(sx), yn = __float2int_rn(sy);
#pragma unroll
                for (int c = 0; c < C; ++c) v[c] = Elem<T>::to_f(tap_global(img + c * plane, k.w, k.h, xn, yn, fillv[c]));
            } else {
                const int x0 = __float2int_rd(sx), y0 = __float2int_rd(sy);
                const float dx = sx - (float)x0, dy = sy - (float)y0;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const T *pl = img + c * plane;
                    const float b4 = blend4(Elem<T>::to_f(tap_global(pl, k.w, k.h, x0, y0, fillv[c])),
                                            Elem<T>::to_f(tap_global(pl, k.w, k.h, x0 + 1, y0, fillv[c])),
                                            Elem<T>::to_f(tap_global(pl, k.w, k.h, x0, y0 + 1, fillv[c])),
                                            Elem<T>::to_f(tap_global(pl, k.w, k.h, x0 + 1, y0 + 1, fillv[c])), dx, dy);
                    v[c] = Elem<T>::to_f(Elem<T>::from_f(b4));
                }
            }
        }
        if (BRIGHT) {
#pragma unroll
            for (int c = 0; c < C; ++c)
                v[c] = sizeof(T) == 4 ? __saturatef(v[c] * bf)
                                      : __saturatef(__half2float(__hmul(__float2half_rn(v[c]), bh)));
        }
        float gr = C == 3 ? 0.2989f * v[0] + 0.587f * v[1] + 0.114f * v[C - 1] : v[0];
        if (sizeof(T) == 2) gr = __half2float(__float2half_rn(gr));
        acc += gr;
    }
    // block sum: shuffle within warps, then across warps through shared memory
    __shared__ float warp_sum[kWarps];
    __shared__ bool is_last;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < kWarps; ++i) s += warp_sum[i];
        partials[(size_t)n * bpi + blk] = s;
        __threadfence();
        is_last = atomicAdd(counters + n, 1u) == (unsigned)(bpi - 1);
    }
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
        __threadfence();
        double s = 0.0;
        for (int i = 0; i < bpi; ++i) s += (double)__ldcg(partials + (size_t)n * bpi + i);
        float m = (float)(s / (double)total);
        if (sizeof(T) == 2) m = __half2float(__float2half_rn(m));
        mean_out[n] = m;
        counters[n] = 0;        // leave the scratch ready for the next call
    }
}

template <typename T, int C, int KIND>
static cudaError_t launch_gray_mean_t(const KArgs &k, bool bright, float *mean_out, unsigned *counters,
                                      float *partials, int bpi, cudaStream_t stream)
{
    dim3 grid(bpi, k.n);
    if (bright) gray_mean_kernel<T, C, KIND, true><<<grid, kThreads, 0, stream>>>(k, mean_out, counters, partials);
    else gray_mean_kernel<T, C, KIND, false><<<grid, kThreads, 0, stream>>>(k, mean_out, counters, partials);
    return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_gray_mean(const KArgs &k, int c, int kind, bool bright, float *mean_out,
                                    unsigned *counters, float *partials, int bpi, cudaStream_t stream)
{
#define TA_GM(CC, KK) launch_gray_mean_t<T, CC, KK>(k, bright, mean_out, counters, partials, bpi, stream)
    if (c == 3) return kind == 0 ? TA_GM(3, 0) : kind == 1 ? TA_GM(3, 1) : TA_GM(3, 2);
    return kind == 0 ? TA_GM(1, 0) : kind == 1 ? TA_GM(1, 1) : TA_GM(1, 2);
#undef TA_GM
}

// ----------------------------------------------------------------------------- staged pre-pass
// fp32 and uint8 images whose rows the tensor copies can read run the pre-pass on the staged kernel
// (REDUCE variant): the same sampling as the fused pass, one partial sum per (tile, consumer
// warp) written to scratch, then one block per image adds that image's partials in a fixed
// order in double.  Measured on 64 x 3 x 1280^2 -> 1024^2: the pre-pass takes 0.24 ms (bilinear)
// / 0.17 ms (nearest) instead of the gather kernel's 0.45 / 0.25 ms.  The gather kernel above
// stays for fp16, unaligned rows and scratch buffers sized for it alone.
// one block of 256 threads per image, one chain each; the order of the additions is chain_sum()'s
// and the tree's, as in mean_of_partials_by_warp()
__global__ void __launch_bounds__(256) mean_finish_kernel(const float *partials, int per_image, int pixels, float *mean_out)
{
    __shared__ double sh[256];
    const int n = blockIdx.x, t = threadIdx.x;
    sh[t] = chain_sum(reinterpret_cast<const float4 *>(partials + (size_t)n * per_image), per_image >> 2, t);
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (t < o) sh[t] += sh[t + o];
        __syncthreads();
    }
    if (t == 0) mean_out[n] = (float)(sh[0] / (double)pixels);
}

static long long mean_staged_tiles(const ta_b200_fused_params *p)
{
    return (long long)p->n * ((p->ow + kTileW - 1) / kTileW) * ((p->oh + kTileH - 1) / kTileH);
}

static bool mean_staged_applicable(const ta_b200_fused_params *p)
{
    if (p->dtype == TA_B200_F16 || p->n <= 0) return false;
    const size_t es = in_bytes(p->dtype);
    if (((size_t)p->w * es) % 16 != 0 || ((uintptr_t)p->in % 16) != 0 || ((size_t)p->h * p->w * es) % 16 != 0) return false;
    if (p->h >= (1 << 22) || p->w >= (1 << 22) || p->oh >= (1 << 22) || p->ow >= (1 << 22)) return false;
    if ((double)p->n * p->c >= 2147483648.0) return false;
    return mean_staged_tiles(p) < (1LL << 24);
}

static size_t mean_gather_need(const ta_b200_fused_params *p)
{
    return mean_partials_offset(p->n) + (size_t)p->n * mean_blocks_per_image(p->oh, p->ow) * sizeof(float);
}
static size_t mean_staged_offset(const ta_b200_fused_params *p) { return (mean_gather_need(p) + 255) / 256 * 256; }
// scratch a caller should pass: the gather kernel's region, then (when applicable) the staged partials
static size_t mean_scratch_need(const ta_b200_fused_params *p)
{
    if (!mean_staged_applicable(p)) return mean_gather_need(p);
    return mean_staged_offset(p) + (size_t)mean_staged_tiles(p) * kConsumerWarps * sizeof(float);
}

static int gray_mean_staged(const ta_b200_fused_params *p, float *mean_out, float *partials, cudaStream_t stream)
{
    DeviceState *s = nullptr;
    int rc = current_device(&s, nullptr);
    if (rc != TA_B200_OK) return rc;
    rc = pending_timeout(*s);
    if (rc != TA_B200_OK) return rc;
    KArgs k;
    fill_kargs(k, p, *s);
    if (!k.staged_ok) return fail(TA_B200_ERR_UNSUPPORTED, "rows cannot be staged");
    const int mode = p->matrix ? (p->interp == TA_B200_BILINEAR ? 2 : 1) : 0;
    const bool bright = (p->apply & TA_B200_APPLY_BRIGHTNESS) != 0;
    const KernelEntry ke = mean_kernel_entry(mode, bright, p->c, in_bytes(p->dtype) == 1);
    int blocks = 0;
    rc = prepare_kernel(*s, ke, 6, p->dtype, p->c, (unsigned)(mode * 2 + (bright ? 1 : 0)), &blocks);
    if (rc != TA_B200_OK) return rc;
    k.out = nullptr;
    k.mean_partials = partials;
    k.late_x_slot = 8;
    if (mode == 0) k.fill[0] = k.fill[1] = k.fill[2] = 0.0f;
    k.tiles_x = (p->ow + kTileW - 1) / kTileW;
    k.tiles_y = (p->oh + kTileH - 1) / kTileH;
    k.num_tiles = (int)mean_staged_tiles(p);
    long long grid = (long long)s->sm_count * blocks;
    if (grid > k.num_tiles) grid = k.num_tiles;
    TMaps maps;
    memset(&maps, 0, sizeof(maps));
    rc = build_tensor_maps(maps, p);
    if (rc != TA_B200_OK) return rc;
    void *args[] = {&k, &maps};
    cudaError_t e = cudaLaunchKernel(ke.fn, dim3((unsigned)grid), dim3(ke.threads), args, ke.smem, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernel(gray_mean, staged)");
    mean_finish_kernel<<<p->n, 256, 0, stream>>>(partials, k.tiles_x * k.tiles_y * kConsumerWarps, p->oh * p->ow, mean_out);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch(mean_finish)");
    return TA_B200_OK;
}

// Checks, scratch carving and launch of the grayscale-mean pre-pass.
static int gray_mean_on(const ta_b200_fused_params *p, float *mean_out, void *scratch, size_t scratch_bytes,
                        cudaStream_t stream, bool clear_counters)
{
    int rc = validate_geometry_only(p);
    if (rc != TA_B200_OK) return rc;
    if (!mean_out) return fail(TA_B200_ERR_NULL, "mean_out is NULL");
    if (p->n == 0) return TA_B200_OK;
    if (p->n > 65535) return fail(TA_B200_ERR_TOO_LARGE, "gray_mean handles at most 65535 images per call");
    const int bpi = mean_blocks_per_image(p->oh, p->ow);
    const size_t need = mean_partials_offset(p->n) + (size_t)p->n * bpi * sizeof(float);
    if (!scratch || scratch_bytes < need || ((uintptr_t)scratch % 256) != 0)
        return fail(TA_B200_ERR_SCRATCH, "scratch must be 256-byte aligned and >= %zu bytes (got %zu)", need,
                    scratch_bytes);
    // a scratch buffer sized by ta_b200_gray_mean_scratch_bytes() has room for the staged kernel's partials
    if (mean_staged_applicable(p) && scratch_bytes >= mean_scratch_need(p))
        return gray_mean_staged(p, mean_out, (float *)((char *)scratch + mean_staged_offset(p)), stream);
    if (in_bytes(p->dtype) == 1)
        return fail(TA_B200_ERR_UNSUPPORTED, "the grayscale mean of a uint8 image needs rows of whole 16-byte units "
                    "(width and plane size multiples of 16, 16-byte aligned base) and %zu bytes of scratch",
                    mean_scratch_need(p));
    DeviceState *s = nullptr;
    rc = current_device(&s, nullptr);
    if (rc != TA_B200_OK) return rc;
    KArgs k;
    fill_kargs(k, p, *s);
    unsigned *counters = (unsigned *)scratch;
    float *partials = (float *)((char *)scratch + mean_partials_offset(p->n));
    cudaError_t e;
    if (clear_counters) {
        e = cudaMemsetAsync(counters, 0, (size_t)p->n * sizeof(unsigned), stream);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(scratch)");
    }
    const int kind = p->matrix ? (p->interp == TA_B200_BILINEAR ? 2 : 1) : 0;
    const bool bright = (p->apply & TA_B200_APPLY_BRIGHTNESS) != 0;
    e = p->dtype == TA_B200_F32
            ? launch_gray_mean<float>(k, p->c, kind, bright, mean_out, counters, partials, bpi, stream)
            : launch_gray_mean<__half>(k, p->c, kind, bright, mean_out, counters, partials, bpi, stream);
    if (e != cudaSuccess) return cuda_fail(e, "launch(gray_mean)");
    return TA_B200_OK;
}

// ----------------------------------------------------------------------------- mean contrast in one call
// ta_b200_fused_augment_mean(): grayscale-mean reduction + fused pass.  By default two launches
// (reduction with its one-warp-per-image finish, then the fused kernel).  ta_b200_mean_path(1 or 2)
// switches to ONE cooperative launch of the two-phase kernel (ta_affine_producer.cuh): the fused
// pass of an image runs one or two images behind its reduction, so its read of the source comes
// from L2 instead of HBM and nothing is launched in between.  Same partial sums, added in the same
// order: identical output either way.  Measured on 64 x 3 x 1280^2 -> 1024^2, all colour
// operations, medians of long runs (power-capped clocks): two launches 467 us nearest / 586 us
// bilinear; one launch 547 / 640 us two images behind, 672 / 745 us one image behind.  Both passes
// are bound by instruction issue, not by HBM, so reading from L2 buys little, while every
// dependency between thread blocks costs: with the mean finished by the consumer warp that happened
// to be last (always the slowest block, made slower still) it was 1100 us, counting partials per
// tile instead of per block and image (8192 additions to one address per image) 2200 us.  Hence
// the default.
static bool two_phase_applicable(const ta_b200_fused_params *p)
{
    if (p->dtype != TA_B200_F32 || !mean_staged_applicable(p)) return false;
    if (late_count_of(p) != 0) return false;                 // the per-pixel recipe has no two-phase build
    return 2 * mean_staged_tiles(p) < 2147483647LL - (1 << 24);
}
static size_t two_phase_partials_offset(int n) { return ((size_t)n * 2 * sizeof(unsigned) + 255) / 256 * 256; }
static size_t two_phase_need(const ta_b200_fused_params *p)
{
    return two_phase_partials_offset(p->n) + (size_t)mean_staged_tiles(p) * kConsumerWarps * sizeof(float);
}

static int fused_mean(const ta_b200_fused_params *p, float *mean_out, void *scratch, size_t scratch_bytes,
                      cudaStream_t stream)
{
    if (!p) return fail(TA_B200_ERR_NULL, "params is NULL");
    const bool mean_mode = (p->apply & TA_B200_APPLY_CONTRAST) && p->contrast_mode == TA_B200_CONTRAST_MEAN;
    if (!mean_mode) return launch_fused(p, stream, false);           // nothing to reduce
    if (!mean_out) return fail(TA_B200_ERR_NULL, "mean_out is NULL");
    ta_b200_fused_params q = *p;
    q.gray_mean = mean_out;
    int rc = validate(&q);
    if (rc != TA_B200_OK) return rc;
    if (p->n == 0) return TA_B200_OK;
    DeviceState *s = nullptr;
    int dev = 0;
    rc = current_device(&s, &dev);
    if (rc != TA_B200_OK) return rc;
    static std::atomic<int> coop[kMaxDevices];                        // 0 unknown, 1 yes, 2 no
    if (coop[dev].load() == 0) {
        int v = 0;
        cudaError_t e = cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev);
        coop[dev].store(e == cudaSuccess && v ? 1 : 2);
    }
    const bool one_launch = g_two_phase.load(std::memory_order_relaxed) != 0 && coop[dev].load() == 1 &&
                            two_phase_applicable(p) && scratch && ((uintptr_t)scratch % 256) == 0 &&
                            scratch_bytes >= two_phase_need(p);
    if (!one_launch) {
        rc = gray_mean_on(p, mean_out, scratch, scratch_bytes, stream, true);
        if (rc != TA_B200_OK) return rc;
        return launch_fused(&q, stream, false);
    }
    rc = pending_timeout(*s);
    if (rc != TA_B200_OK) return rc;
    KArgs k;
    fill_kargs(k, &q, *s);
    if (!k.staged_ok) return fail(TA_B200_ERR_UNSUPPORTED, "rows cannot be staged");
    const int mode = p->matrix ? (p->interp == TA_B200_BILINEAR ? 2 : 1) : 0;
    if (mode == 0) k.fill[0] = k.fill[1] = k.fill[2] = 0.0f;
    const unsigned f = template_flags(&q);
    const KernelTable &tab = table_f32_two_phase(mode);
    const KernelEntry *ke = p->c == 3 ? &tab.c3[f] : &tab.c1[f];
    if (!ke->fn) return fail(TA_B200_ERR_UNSUPPORTED, "no two-phase kernel for channels=%d flags=0x%x", p->c, f);
    int blocks = 0;
    rc = prepare_kernel(*s, *ke, 7 + mode, p->dtype, p->c, f, &blocks);
    if (rc != TA_B200_OK) return rc;
    k.tiles_x = (p->ow + kTileW - 1) / kTileW;
    k.tiles_y = (p->oh + kTileH - 1) / kTileH;
    k.num_tiles = (int)(2 * mean_staged_tiles(p));
    k.mean_done = (unsigned *)scratch;
    k.mean_ready = k.mean_done + p->n;
    k.mean_partials = (float *)((char *)scratch + two_phase_partials_offset(p->n));
    k.mean_out = mean_out;
    k.mean_pixels = p->oh * p->ow;
    k.mean_lag = g_two_phase.load(std::memory_order_relaxed) >= 2 ? 2 : 1;
    // every CTA must be resident at once (CTAs wait for one another's partial sums): one wave at most
    long long grid = (long long)s->sm_count * blocks;
    if (grid > k.num_tiles) grid = k.num_tiles;
    TMaps maps;
    memset(&maps, 0, sizeof(maps));
    rc = build_tensor_maps(maps, p);
    if (rc != TA_B200_OK) return rc;
    cudaError_t e = cudaMemsetAsync(scratch, 0, two_phase_partials_offset(p->n), stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(two-phase counters)");
    void *args[] = {&k, &maps};
    e = cudaLaunchCooperativeKernel(ke->fn, dim3((unsigned)grid), dim3(ke->threads), args, ke->smem, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchCooperativeKernel(two-phase)");
    return TA_B200_OK;
}

// ----------------------------------------------------------------------------- inverse affine matrices
// Every operation individually rounded, in the order of triton_augment/functional.py:853-890
// (which runs each line as its own elementwise op).
__device__ __forceinline__ void inverse_matrix_of(float angle, float tx, float ty, float sc, float shear_x, float shear_y,
                                                  float cx, float cy, float *m)
{
    const float d2r = (float)(3.141592653589793 / 180.0);
    const float rot = __fmul_rn(angle, d2r);
    const float sx = __fmul_rn(shear_x, d2r), sy = __fmul_rn(shear_y, d2r);
    const float cos_sy = cosf(sy);
    const float rms = __fsub_rn(rot, sy);
    const float a = __fdiv_rn(cosf(rms), cos_sy);
    const float b = __fsub_rn(__fdiv_rn(__fmul_rn(-cosf(rms), tanf(sx)), cos_sy), sinf(rot));
    const float c = __fdiv_rn(sinf(rms), cos_sy);
    const float d = __fadd_rn(__fdiv_rn(__fmul_rn(-sinf(rms), tanf(sx)), cos_sy), cosf(rot));
    const float m0 = __fdiv_rn(d, sc), m1 = __fdiv_rn(-b, sc), m3 = __fdiv_rn(-c, sc), m4 = __fdiv_rn(a, sc);
    const float ux = __fsub_rn(-cx, tx), uy = __fsub_rn(-cy, ty);
    float m2 = __fadd_rn(__fmul_rn(m0, ux), __fmul_rn(m1, uy));
    float m5 = __fadd_rn(__fmul_rn(m3, ux), __fmul_rn(m4, uy));
    m2 = __fadd_rn(m2, cx);
    m5 = __fadd_rn(m5, cy);
    m[0] = m0; m[1] = m1; m[2] = m2; m[3] = m3; m[4] = m4; m[5] = m5;
}

// One thread per image.
__global__ void inverse_matrix_kernel(int n, const float *center, const float *angle, const float *translate,
                                      const float *scale, const float *shear, float *matrix)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    inverse_matrix_of(angle[i], translate[2 * i], translate[2 * i + 1], scale[i], shear[2 * i], shear[2 * i + 1],
                      center ? center[2 * i] : 0.0f, center ? center[2 * i + 1] : 0.0f, matrix + 6 * (size_t)i);
}

// ----------------------------------------------------------------------------- fused parameter sampler
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11): a
// counter-based generator, so the parameter set p of a call is a pure function of (seed, p)
// and samples that share a parameter set simply compute it again.
__device__ __forceinline__ uint4 philox4x32_10(uint2 key, uint4 ctr)
{
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
        ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
        key.x += 0x9E3779B9u;
        key.y += 0xBB67AE85u;
    }
    return ctr;
}

__device__ __forceinline__ float unit_float(uint32_t bits) { return (float)(bits >> 8) * (1.0f / 16777216.0f); }   // [0, 1)
__device__ __forceinline__ float uniform_in(uint32_t bits, const float (&r)[2]) { return r[0] == r[1] ? r[0] : r[0] + unit_float(bits) * (r[1] - r[0]); }

__global__ void store_words_kernel(uint64_t *dst, uint64_t a, uint64_t b) { dst[0] = a; dst[1] = b; }

// ---- PyTorch's CUDA generator, restated (ATen/native/cuda/DistributionTemplates.h, curand's Philox
// state: curand_philox4x32_x.h).  A draw of `numel` values launches ceil(numel / 256) blocks of 256
// threads (at most SM count x resident blocks); thread t starts curand at (seed, subsequence t,
// offset) and, while numel <= the thread count, value t is made from the first word of its first
// four-word block, i.e. Philox(key = seed, counter = (offset / 4 lo, hi, t lo, t hi)).x.
__device__ __forceinline__ uint32_t torch_word(uint64_t seed, uint64_t offset4, uint32_t draw, uint32_t index)
{
    const uint64_t c = offset4 + draw;
    return philox4x32_10(make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)),
                         make_uint4((uint32_t)c, (uint32_t)(c >> 32), index, 0u)).x;
}
// curand_uniform: word -> (0, 1]
__device__ __forceinline__ float torch_unit(uint32_t w, bool fused)
{
    const float x = __uint2float_rn(w), k = 2.3283064e-10f, h = 2.3283064e-10f / 2.0f;
    return fused ? __fmaf_rn(x, k, h) : __fadd_rn(__fmul_rn(x, k), h);
}
// tensor.uniform_(from, to): rand * (to - from) + from, the value `to` folded back to `from`
__device__ __forceinline__ float torch_uniform(uint32_t w, float from, float to, int flags)
{
    const float r = torch_unit(w, (flags & 2) != 0), range = __fsub_rn(to, from);
    const float v = (flags & 4) ? __fmaf_rn(r, range, from) : __fadd_rn(__fmul_rn(r, range), from);
    return v == to ? from : v;
}

template <typename FT>
__global__ void sample_params_kernel(const __grid_constant__ ta_b200_sample_spec s)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= s.total) return;
    const int gi = s.first_sample + i;                   // the sample's index in the whole batch
    int p;
    if (s.frames <= 1) p = s.same_on_batch ? 0 : gi;
    else p = (s.same_on_batch ? 0 : gi / s.frames) * (s.same_on_frame ? 1 : s.frames) + (s.same_on_frame ? 0 : gi % s.frames);
    if (s.torch_compat) {
        const uint64_t seed = s.torch_state ? s.torch_state[0] : s.torch_seed;
        const uint64_t off4 = (s.torch_state ? s.torch_state[1] : s.torch_offset) >> 2;
        const int fl = s.torch_compat;
        auto word = [&](int j) { return torch_word(seed, off4, (uint32_t)s.draw[j], (uint32_t)p); };
        auto uni = [&](int j, float lo, float hi, float neutral) { return s.draw[j] < 0 ? neutral : torch_uniform(word(j), lo, hi, fl); };
        const float max_dx = s.translate[0], max_dy = s.translate[1];        // pixels in this mode
        const float angle = uni(0, s.degrees[0], s.degrees[1], 0.0f);
        const float tx = uni(1, -max_dx, max_dx, 0.0f), ty = uni(2, -max_dy, max_dy, 0.0f);
        const float sc = uni(3, s.scale[0], s.scale[1], 1.0f);
        const float shx = uni(4, s.shear[0], s.shear[1], 0.0f), shy = uni(5, s.shear[2], s.shear[3], 0.0f);
        if (s.matrix) inverse_matrix_of(angle, tx, ty, sc, shx, shy, 0.0f, 0.0f, s.matrix + 6 * (size_t)i);
        if (s.angle_out) s.angle_out[i] = angle;
        if (s.translate_out) { s.translate_out[2 * i] = tx; s.translate_out[2 * i + 1] = ty; }
        if (s.scale_out) s.scale_out[i] = sc;
        if (s.shear_out) { s.shear_out[2 * i] = shx; s.shear_out[2 * i + 1] = shy; }
        // randint(0, size - crop + 1): word % range (ATen/core/TransformationHelper.h, uniform_int_from_to)
        const uint32_t span_y = (uint32_t)(s.img_h - s.crop_h + 1), span_x = (uint32_t)(s.img_w - s.crop_w + 1);
        if (s.top) s.top[i] = s.draw[6] < 0 ? 0.0f : (float)(word(6) % span_y);
        if (s.left) s.left[i] = s.draw[7] < 0 ? 0.0f : (float)(word(7) % span_x);
        // rand(n) < p
        if (s.flip) s.flip[i] = s.draw[8] >= 0 && torch_uniform(word(8), 0.0f, 1.0f, fl) < s.flip_p ? 1 : 0;
        if (s.brightness_out) ((FT *)s.brightness_out)[i] = (FT)uni(9, s.brightness[0], s.brightness[1], 1.0f);
        if (s.contrast_out) ((FT *)s.contrast_out)[i] = (FT)uni(10, s.contrast[0], s.contrast[1], 1.0f);
        if (s.saturation_out) ((FT *)s.saturation_out)[i] = (FT)uni(11, s.saturation[0], s.saturation[1], 1.0f);
        if (s.gray) s.gray[i] = s.draw[12] >= 0 && torch_uniform(word(12), 0.0f, 1.0f, fl) < s.grayscale_p ? 1 : 0;
        return;
    }
    const uint64_t seed = *s.seed;
    const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
    uint32_t u[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 v = philox4x32_10(key, make_uint4((uint32_t)p, 0u, (uint32_t)j, 0x7461b200u));
        u[4 * j] = v.x; u[4 * j + 1] = v.y; u[4 * j + 2] = v.z; u[4 * j + 3] = v.w;
    }
    const float angle = uniform_in(u[0], s.degrees);
    const float tr_x[2] = {-s.translate[0] * (float)s.img_w, s.translate[0] * (float)s.img_w};
    const float tr_y[2] = {-s.translate[1] * (float)s.img_h, s.translate[1] * (float)s.img_h};
    const float tx = uniform_in(u[1], tr_x), ty = uniform_in(u[2], tr_y);
    const float sc = uniform_in(u[3], s.scale);
    const float sh_x[2] = {s.shear[0], s.shear[1]}, sh_y[2] = {s.shear[2], s.shear[3]};
    const float shx = uniform_in(u[4], sh_x), shy = uniform_in(u[5], sh_y);
    if (s.matrix) inverse_matrix_of(angle, tx, ty, sc, shx, shy, 0.0f, 0.0f, s.matrix + 6 * (size_t)i);
    if (s.angle_out) s.angle_out[i] = angle;
    if (s.translate_out) { s.translate_out[2 * i] = tx; s.translate_out[2 * i + 1] = ty; }
    if (s.scale_out) s.scale_out[i] = sc;
    if (s.shear_out) { s.shear_out[2 * i] = shx; s.shear_out[2 * i + 1] = shy; }
    // crop offsets: integers in [0, size - crop], as floats (what the fused kernel takes)
    const int span_y = s.crop_h > 0 ? s.img_h - s.crop_h + 1 : 1, span_x = s.crop_w > 0 ? s.img_w - s.crop_w + 1 : 1;
    if (s.top) s.top[i] = (float)min((int)(unit_float(u[6]) * (float)span_y), span_y - 1);
    if (s.left) s.left[i] = (float)min((int)(unit_float(u[7]) * (float)span_x), span_x - 1);
    if (s.flip) s.flip[i] = unit_float(u[8]) < s.flip_p ? 1 : 0;
    if (s.brightness_out) ((FT *)s.brightness_out)[i] = (FT)uniform_in(u[9], s.brightness);
    if (s.contrast_out) ((FT *)s.contrast_out)[i] = (FT)uniform_in(u[10], s.contrast);
    if (s.saturation_out) ((FT *)s.saturation_out)[i] = (FT)uniform_in(u[11], s.saturation);
    if (s.gray) s.gray[i] = unit_float(u[12]) < s.grayscale_p ? 1 : 0;
}

}  // namespace ta

#include "ta_api_host.cuh"
