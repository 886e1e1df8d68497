// Third part of ta_api.cu: the host-buffer pipeline and the extern "C" functions.
#pragma once

namespace ta {

// ----------------------------------------------------------------------------- host-buffer pipeline
// Images are independent, so a host batch is cut into slices; slice i uploads while
// slice i-1 runs and slice i-2 downloads.  Two input and two output device buffers per
// device, three streams, events between them.  Buffers and streams are created on first
// use and kept (grown when a later call needs more).
struct HostPipe {
    std::mutex mu;
    bool ready = false;
    cudaStream_t up = nullptr, run = nullptr, down = nullptr;
    cudaEvent_t uploaded[2] = {}, computed[2] = {}, downloaded[2] = {};
    void *d_in[2] = {}, *d_out[2] = {};
    size_t in_cap = 0, out_cap = 0;
    void *d_params = nullptr;
    size_t params_cap = 0;
    void *d_scratch = nullptr;
    size_t scratch_cap = 0;
};
static HostPipe g_pipe[kMaxDevices];
// ta_b200_debug_host_upload(): 0 whole images always, 1 per-image boxes where they pay, 2 boxes
// whenever the images are large enough (tests compare them)
static std::atomic<int> g_host_trim{1};

static cudaError_t grow(void **ptr, size_t *cap, size_t need)
{
    if (need <= *cap) return cudaSuccess;
    if (*ptr) { cudaError_t e = cudaFree(*ptr); if (e != cudaSuccess) return e; *ptr = nullptr; *cap = 0; }
    cudaError_t e = cudaMalloc(ptr, need);
    if (e == cudaSuccess) *cap = need;
    return e;
}

// The part of source image `i` that a call reads, as a box [x0, x1) x [y0, y1) clipped to the
// image: the host-buffer path uploads nothing else.  The map output pixel -> source position is
// affine (triton_augment/kernels/geometric_kernel.py:386-415), so the extreme positions belong
// to the four corners of the output; two pixels of margin cover the taps of either sampling
// mode (rint, or floor and floor + 1, zero-weight taps included) and the float32 evaluation in
// the kernels.  Coordinates that are not finite or huge give the whole image.
static void source_box(const ta_b200_fused_params *hp, int i, int &x0, int &x1, int &y0, int &y1)
{
    x0 = 0; x1 = hp->w; y0 = 0; y1 = hp->h;
    const double left = hp->left ? (double)hp->left[i] : 0.0, top = hp->top ? (double)hp->top[i] : 0.0;
    const double xa = left, xb = left + (hp->ow - 1), ya = top, yb = top + (hp->oh - 1);
    double xmin, xmax, ymin, ymax;
    if (hp->matrix) {
        const float *m = hp->matrix + (size_t)i * 6;
        const double hw = 0.5 * hp->w, hh = 0.5 * hp->h;
        xmin = ymin = INFINITY; xmax = ymax = -INFINITY;
        for (int k = 0; k < 4; ++k) {
            const double xc = ((k & 1) ? xb : xa) - hw + 0.5, yc = ((k & 2) ? yb : ya) - hh + 0.5;
            const double sx = (double)m[0] * xc + (double)m[1] * yc + (double)m[2] + hw - 0.5;
            const double sy = (double)m[3] * xc + (double)m[4] * yc + (double)m[5] + hh - 0.5;
            if (!(fabs(sx) < 1.0e6) || !(fabs(sy) < 1.0e6)) return;
            xmin = fmin(xmin, sx); xmax = fmax(xmax, sx); ymin = fmin(ymin, sy); ymax = fmax(ymax, sy);
        }
    } else {
        if (!(fabs(xa) < 1.0e6) || !(fabs(ya) < 1.0e6)) return;
        xmin = xa; xmax = xb; ymin = ya; ymax = yb;
    }
    const long long bx0 = (long long)floor(xmin) - 2, bx1 = (long long)ceil(xmax) + 3;
    const long long by0 = (long long)floor(ymin) - 2, by1 = (long long)ceil(ymax) + 3;
    x0 = (int)(bx0 < 0 ? 0 : bx0 > hp->w ? hp->w : bx0);
    x1 = (int)(bx1 < 0 ? 0 : bx1 > hp->w ? hp->w : bx1);
    y0 = (int)(by0 < 0 ? 0 : by0 > hp->h ? hp->h : by0);
    y1 = (int)(by1 < 0 ? 0 : by1 > hp->h ? hp->h : by1);
}

#define TA_CU(call, what) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return cuda_fail(e_, what); } while (0)

// Whatever way fused_host() is left, nothing it enqueued may still be running: copies read and
// write the caller's host buffers, and the next call reuses the device buffers without waiting.
struct DrainPipe {
    HostPipe &P;
    explicit DrainPipe(HostPipe &p) : P(p) {}
    ~DrainPipe()
    {
        if (P.up) cudaStreamSynchronize(P.up);
        if (P.run) cudaStreamSynchronize(P.run);
        if (P.down) cudaStreamSynchronize(P.down);
    }
};

static int fused_host(const ta_b200_fused_params *hp)
{
    // Validate with the device checks relaxed: gray_mean may be computed here.
    ta_b200_fused_params v = *hp;
    static const float dummy = 0.0f;
    const bool need_mean = (hp->apply & TA_B200_APPLY_CONTRAST) && hp->contrast_mode == TA_B200_CONTRAST_MEAN;
    if (need_mean && !v.gray_mean) v.gray_mean = &dummy;
    int rc = validate(&v);
    if (rc != TA_B200_OK) return rc;
    if (hp->n == 0) return TA_B200_OK;
    DeviceState *s = nullptr;
    int dev = 0;
    rc = current_device(&s, &dev);
    if (rc != TA_B200_OK) return rc;
    HostPipe &P = g_pipe[dev];
    std::lock_guard<std::mutex> lock(P.mu);
    if (!P.ready) {
        TA_CU(cudaStreamCreateWithFlags(&P.up, cudaStreamNonBlocking), "cudaStreamCreate");
        TA_CU(cudaStreamCreateWithFlags(&P.run, cudaStreamNonBlocking), "cudaStreamCreate");
        TA_CU(cudaStreamCreateWithFlags(&P.down, cudaStreamNonBlocking), "cudaStreamCreate");
        for (int i = 0; i < 2; ++i) {
            TA_CU(cudaEventCreateWithFlags(&P.uploaded[i], cudaEventDisableTiming), "cudaEventCreate");
            TA_CU(cudaEventCreateWithFlags(&P.computed[i], cudaEventDisableTiming), "cudaEventCreate");
            TA_CU(cudaEventCreateWithFlags(&P.downloaded[i], cudaEventDisableTiming), "cudaEventCreate");
        }
        P.ready = true;
    }
    rc = pending_timeout(*s);
    if (rc != TA_B200_OK) return rc;
    DrainPipe drain(P);          // every exit below, failures included, waits for the three streams
    const size_t es = ta::out_bytes(hp->dtype);          // output elements and factor vectors
    const size_t in_img = (size_t)hp->c * hp->h * hp->w * ta::in_bytes(hp->dtype), out_img = (size_t)hp->c * hp->oh * hp->ow * es;
    // Slice size: about 48 MiB of input per slice, at least 1 image, at least 4 slices when possible.
    long long per = (long long)((48ull << 20) / (in_img ? in_img : 1));
    if (per < 1) per = 1;
    if (per > (hp->n + 3) / 4) per = (hp->n + 3) / 4;
    if (per < 1) per = 1;
    const int slice = (int)per;
    // d_in[0]/d_in[1] share one capacity value: grow both when needed.
    if ((size_t)slice * in_img > P.in_cap) {
        for (int i = 0; i < 2; ++i) {
            if (P.d_in[i]) TA_CU(cudaFree(P.d_in[i]), "cudaFree");
            P.d_in[i] = nullptr;
            TA_CU(cudaMalloc(&P.d_in[i], (size_t)slice * in_img), "cudaMalloc(input slice)");
        }
        P.in_cap = (size_t)slice * in_img;
    }
    if ((size_t)slice * out_img > P.out_cap) {
        for (int i = 0; i < 2; ++i) {
            if (P.d_out[i]) TA_CU(cudaFree(P.d_out[i]), "cudaFree");
            P.d_out[i] = nullptr;
            TA_CU(cudaMalloc(&P.d_out[i], (size_t)slice * out_img), "cudaMalloc(output slice)");
        }
        P.out_cap = (size_t)slice * out_img;
    }
    // Per-image parameters: one device block, each vector 256-byte aligned.
    const size_t n = (size_t)hp->n;
    auto al = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t o_top = 0, o_left = o_top + al(n * 4), o_flip = o_left + al(n * 4), o_mat = o_flip + al(n),
                 o_b = o_mat + al(n * 24), o_c = o_b + al(n * es), o_s = o_c + al(n * es), o_g = o_s + al(n * es),
                 o_gm = o_g + al(n), total = o_gm + al(n * 4);
    TA_CU(grow(&P.d_params, &P.params_cap, total), "cudaMalloc(params)");
    char *dp = (char *)P.d_params;
    auto up = [&](const void *src, size_t off, size_t bytes) -> cudaError_t {
        return src ? cudaMemcpyAsync(dp + off, src, bytes, cudaMemcpyHostToDevice, P.run) : cudaSuccess;
    };
    TA_CU(up(hp->top, o_top, n * 4), "upload top");
    TA_CU(up(hp->left, o_left, n * 4), "upload left");
    TA_CU(up(hp->flip, o_flip, n), "upload flip");
    TA_CU(up(hp->matrix, o_mat, n * 24), "upload matrix");
    TA_CU(up(hp->brightness, o_b, n * es), "upload brightness");
    TA_CU(up(hp->contrast, o_c, n * es), "upload contrast");
    TA_CU(up(hp->saturation, o_s, n * es), "upload saturation");
    TA_CU(up(hp->gray, o_g, n), "upload gray");
    if (need_mean && hp->gray_mean) TA_CU(up(hp->gray_mean, o_gm, n * 4), "upload gray_mean");
    if (need_mean && !hp->gray_mean) {
        ta_b200_fused_params one = *hp;          // a slice: device input at a 256-byte aligned address
        one.n = slice;
        one.in = P.d_in[0];
        // decided for the whole call before the first copy is enqueued
        if (ta::in_bytes(hp->dtype) == 1 && !mean_staged_applicable(&one))
            return fail(TA_B200_ERR_UNSUPPORTED, "the grayscale mean of a uint8 image needs rows of whole 16-byte units "
                        "(width and plane size multiples of 16)");
        TA_CU(grow(&P.d_scratch, &P.scratch_cap, mean_scratch_need(&one)), "cudaMalloc(scratch)");
    }

    // Upload plan.  Of a large image only the box that is read needs to go up, as one copy per
    // image: either its rows whole (a run of bytes per channel) or the box itself (strided).
    // Measured with pinned batches: a strided copy moves rows of 2-4 KB at about 0.6 of the 50 GB/s
    // of a contiguous one (shorter rows: less), and a separate copy per image costs up to as much
    // as 1 MB of payload.  With those two figures the plan is priced per image, and the call uses
    // it only when it undercuts the plain slice copies by 10 % (128 x 3 x 1024^2 -> 512^2 float32
    // crops: 30.1 ms -> 12.7-13.0 ms; 64 x 3 x 1280^2 -> 1024^2 crops: 24.8 -> 22.1-22.5 ms; the same
    // with +-15 degrees reads nearly every row, gained 2-6 % on float32 and lost 6 % on bytes when
    // forced, and keeps the plain copies).
    const size_t es_in = ta::in_bytes(hp->dtype), row_bytes = (size_t)hp->w * es_in, plane_bytes = row_bytes * hp->h;
    const int col_unit = (int)(32 / es_in);
    struct Box { int x0, x1, y0, y1; bool strided; };
    std::vector<Box> boxes;
    bool trim = g_host_trim.load(std::memory_order_relaxed) != 0 && plane_bytes >= (1u << 20);
    if (trim) {
        boxes.resize((size_t)hp->n);
        const double per_copy = 1.0e6;
        double planned = 0.0;
        for (int i = 0; i < hp->n; ++i) {
            Box &bx = boxes[(size_t)i];
            source_box(hp, i, bx.x0, bx.x1, bx.y0, bx.y1);
            bx.strided = false;
            if (bx.x1 <= bx.x0 || bx.y1 <= bx.y0) { bx.x0 = bx.x1 = 0; continue; }     // nothing of this image is read
            bx.x0 = bx.x0 / col_unit * col_unit;                                        // 32-byte units
            bx.x1 = (bx.x1 + col_unit - 1) / col_unit * col_unit;
            if (bx.x1 > hp->w) bx.x1 = hp->w;
            const double rows_cost = (double)hp->c * (bx.y1 - bx.y0) * (double)row_bytes;
            const double box_bytes = (double)hp->c * (bx.y1 - bx.y0) * (double)(bx.x1 - bx.x0) * (double)es_in;
            bx.strided = (size_t)(bx.x1 - bx.x0) * es_in >= 2048 && box_bytes / 0.6 < rows_cost;
            if (!bx.strided) { bx.x0 = 0; bx.x1 = hp->w; }
            planned += per_copy + (bx.strided ? box_bytes / 0.6 : rows_cost);
        }
        trim = planned <= 0.90 * (double)hp->n * (double)in_img || g_host_trim.load(std::memory_order_relaxed) == 2;
    }
    const int slices = (hp->n + slice - 1) / slice;
    for (int i = 0; i < slices; ++i) {
        const int b = i & 1, first = i * slice, cnt = (first + slice <= hp->n) ? slice : hp->n - first;
        // upload: the input buffer is free once the kernel of slice i-2 has run
        if (i >= 2) TA_CU(cudaStreamWaitEvent(P.up, P.computed[b], 0), "cudaStreamWaitEvent");
        if (!trim) {
            TA_CU(cudaMemcpyAsync(P.d_in[b], (const char *)hp->in + (size_t)first * in_img, (size_t)cnt * in_img,
                                  cudaMemcpyHostToDevice, P.up), "cudaMemcpyAsync(upload)");
        } else {
            // the rest of the device buffer keeps stale bytes, which no kernel reads
            for (int j = 0; j < cnt; ++j) {
                const Box &bx = boxes[(size_t)(first + j)];
                if (bx.x1 <= bx.x0) continue;
                char *dst_img = (char *)P.d_in[b] + (size_t)j * in_img;
                const char *src_img = (const char *)hp->in + (size_t)(first + j) * in_img;
                if (!bx.strided) {
                    // rows y0..y1 of every channel: c runs of bytes, plane_bytes apart
                    const size_t at = (size_t)bx.y0 * row_bytes;
                    TA_CU(cudaMemcpy2DAsync(dst_img + at, plane_bytes, src_img + at, plane_bytes, (size_t)(bx.y1 - bx.y0) * row_bytes,
                                            (size_t)hp->c, cudaMemcpyHostToDevice, P.up), "cudaMemcpy2DAsync(upload rows)");
                } else {
                    cudaMemcpy3DParms cp;
                    memset(&cp, 0, sizeof(cp));
                    cp.srcPtr = make_cudaPitchedPtr(const_cast<char *>(src_img), row_bytes, row_bytes, (size_t)hp->h);
                    cp.dstPtr = make_cudaPitchedPtr(dst_img, row_bytes, row_bytes, (size_t)hp->h);
                    cp.srcPos = cp.dstPos = make_cudaPos((size_t)bx.x0 * es_in, (size_t)bx.y0, 0);
                    cp.extent = make_cudaExtent((size_t)(bx.x1 - bx.x0) * es_in, (size_t)(bx.y1 - bx.y0), (size_t)hp->c);
                    cp.kind = cudaMemcpyHostToDevice;
                    TA_CU(cudaMemcpy3DAsync(&cp, P.up), "cudaMemcpy3DAsync(upload box)");
                }
            }
        }
        TA_CU(cudaEventRecord(P.uploaded[b], P.up), "cudaEventRecord");
        // run: needs its upload, and its output buffer back from the download of slice i-2
        TA_CU(cudaStreamWaitEvent(P.run, P.uploaded[b], 0), "cudaStreamWaitEvent");
        if (i >= 2) TA_CU(cudaStreamWaitEvent(P.run, P.downloaded[b], 0), "cudaStreamWaitEvent");
        ta_b200_fused_params q = *hp;
        q.n = cnt;
        q.in = P.d_in[b];
        q.out = P.d_out[b];
        q.top = hp->top ? (const float *)(dp + o_top) + first : nullptr;
        q.left = hp->left ? (const float *)(dp + o_left) + first : nullptr;
        q.flip = hp->flip ? (const uint8_t *)(dp + o_flip) + first : nullptr;
        q.matrix = hp->matrix ? (const float *)(dp + o_mat) + (size_t)first * 6 : nullptr;
        q.brightness = hp->brightness ? dp + o_b + (size_t)first * es : nullptr;
        q.contrast = hp->contrast ? dp + o_c + (size_t)first * es : nullptr;
        q.saturation = hp->saturation ? dp + o_s + (size_t)first * es : nullptr;
        q.gray = hp->gray ? (const uint8_t *)(dp + o_g) + first : nullptr;
        q.gray_mean = need_mean ? (const float *)(dp + o_gm) + first : nullptr;
        if (need_mean && !hp->gray_mean) {
            rc = gray_mean_on(&q, (float *)(dp + o_gm) + first, P.d_scratch, P.scratch_cap, P.run, true);
            if (rc != TA_B200_OK) return rc;
        }
        rc = launch_fused(&q, P.run, false, (unsigned)first);
        if (rc != TA_B200_OK) return rc;
        TA_CU(cudaEventRecord(P.computed[b], P.run), "cudaEventRecord");
        // download
        TA_CU(cudaStreamWaitEvent(P.down, P.computed[b], 0), "cudaStreamWaitEvent");
        TA_CU(cudaMemcpyAsync((char *)hp->out + (size_t)first * out_img, P.d_out[b], (size_t)cnt * out_img,
                              cudaMemcpyDeviceToHost, P.down), "cudaMemcpyAsync(download)");
        TA_CU(cudaEventRecord(P.downloaded[b], P.down), "cudaEventRecord");
    }
    TA_CU(cudaStreamSynchronize(P.down), "cudaStreamSynchronize");
    TA_CU(cudaStreamSynchronize(P.run), "cudaStreamSynchronize");
    TA_CU(cudaStreamSynchronize(P.up), "cudaStreamSynchronize");
    return pending_timeout(*s);          // a slice whose kernel gave up left p->out incomplete
}

// Streams, events and device buffers of the host-buffer pipeline on the current device.
static int host_release()
{
    int dev = -1;
    TA_CU(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(TA_B200_ERR_DEVICE, "device index %d not supported", dev);
    HostPipe &P = g_pipe[dev];
    std::lock_guard<std::mutex> lock(P.mu);
    { DrainPipe drain(P); }
    for (int i = 0; i < 2; ++i) {
        if (P.d_in[i]) TA_CU(cudaFree(P.d_in[i]), "cudaFree");
        if (P.d_out[i]) TA_CU(cudaFree(P.d_out[i]), "cudaFree");
        P.d_in[i] = P.d_out[i] = nullptr;
        if (P.uploaded[i]) cudaEventDestroy(P.uploaded[i]);
        if (P.computed[i]) cudaEventDestroy(P.computed[i]);
        if (P.downloaded[i]) cudaEventDestroy(P.downloaded[i]);
        P.uploaded[i] = P.computed[i] = P.downloaded[i] = nullptr;
    }
    if (P.d_params) TA_CU(cudaFree(P.d_params), "cudaFree");
    if (P.d_scratch) TA_CU(cudaFree(P.d_scratch), "cudaFree");
    P.d_params = P.d_scratch = nullptr;
    P.in_cap = P.out_cap = P.params_cap = P.scratch_cap = 0;
    if (P.up) cudaStreamDestroy(P.up);
    if (P.run) cudaStreamDestroy(P.run);
    if (P.down) cudaStreamDestroy(P.down);
    P.up = P.run = P.down = nullptr;
    P.ready = false;
    return TA_B200_OK;
}

}  // namespace ta

// ----------------------------------------------------------------------------- C ABI
extern "C" {

int ta_b200_abi_version(void) { return TA_B200_ABI_VERSION; }

const char *ta_b200_last_error(void) { return ta::g_err; }

int ta_b200_fused_augment(const ta_b200_fused_params *p, void *stream)
{
    return ta::launch_fused(ta::Imported(p).ptr, (cudaStream_t)stream, false);
}

int ta_b200_fused_augment_at(const ta_b200_fused_params *p, uint32_t first_image, void *stream)
{
    return ta::launch_fused(ta::Imported(p).ptr, (cudaStream_t)stream, false, first_image);
}

size_t ta_b200_gray_mean_scratch_bytes(const ta_b200_fused_params *p)
{
    if (!p || p->n <= 0 || p->oh <= 0 || p->ow <= 0) return 256;
    return ta::mean_scratch_need(ta::Imported(p).ptr);
}

int ta_b200_gray_mean(const ta_b200_fused_params *p, float *mean_out, void *scratch, size_t scratch_bytes,
                      void *stream)
{
    return ta::gray_mean_on(ta::Imported(p).ptr, mean_out, scratch, scratch_bytes, (cudaStream_t)stream, true);
}

int ta_b200_fused_augment_mean(const ta_b200_fused_params *p, float *mean_out, void *scratch, size_t scratch_bytes,
                               void *stream)
{
    return ta::fused_mean(ta::Imported(p).ptr, mean_out, scratch, scratch_bytes, (cudaStream_t)stream);
}

size_t ta_b200_fused_augment_mean_scratch_bytes(const ta_b200_fused_params *p)
{
    if (!p || p->n <= 0 || p->oh <= 0 || p->ow <= 0) return 256;
    ta::Imported imp(p);
    const ta_b200_fused_params *q = imp.ptr;
    size_t need = ta::mean_scratch_need(q);
    if (ta::two_phase_applicable(q) && ta::two_phase_need(q) > need) need = ta::two_phase_need(q);
    return need;
}

int ta_b200_mean_path(int32_t one_launch)
{
    ta::g_two_phase.store(one_launch < 0 ? 0 : one_launch > 2 ? 2 : one_launch, std::memory_order_relaxed);
    return TA_B200_OK;
}

int ta_b200_fused_augment_host(const ta_b200_fused_params *p) { return p ? ta::fused_host(ta::Imported(p).ptr) : ta::fail(TA_B200_ERR_NULL, "params is NULL"); }

int ta_b200_host_release(void) { return ta::host_release(); }

int ta_b200_status(int acknowledge)
{
    ta::DeviceState *s = nullptr;
    int rc = ta::current_device(&s, nullptr);
    if (rc != TA_B200_OK) return rc;
    rc = ta::pending_timeout(*s);
    if (rc != TA_B200_OK && acknowledge) *(volatile unsigned *)s->status = 0u;
    return rc;
}

int ta_b200_debug_wait(uint64_t limit_ns, int32_t skip_arrive_tile)
{
    ta::g_wait_ns.store(limit_ns ? (unsigned long long)limit_ns : ta::kDefaultWaitNs, std::memory_order_relaxed);
    ta::g_skip_arrive_tile.store(skip_arrive_tile, std::memory_order_relaxed);
    return TA_B200_OK;
}

int ta_b200_debug_host_upload(int32_t trimmed)
{
    if (trimmed < 0 || trimmed > 2) return ta::fail(TA_B200_ERR_UNSUPPORTED, "mode %d", trimmed);
    ta::g_host_trim.store(trimmed, std::memory_order_relaxed);
    return TA_B200_OK;
}

int ta_b200_inverse_affine_matrix(int32_t n, const float *center, const float *angle, const float *translate,
                                  const float *scale, const float *shear, float *matrix, void *stream)
{
    if (n < 0) return ta::fail(TA_B200_ERR_SHAPE, "n = %d", n);
    if (n == 0) return TA_B200_OK;
    if (!angle || !translate || !scale || !shear || !matrix) return ta::fail(TA_B200_ERR_NULL, "NULL argument");
    ta::inverse_matrix_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(n, center, angle, translate, scale,
                                                                                 shear, matrix);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ta::cuda_fail(e, "launch(inverse_matrix)");
    return TA_B200_OK;
}

int ta_b200_sample_params(const ta_b200_sample_spec *spec, void *stream)
{
    if (!spec) return ta::fail(TA_B200_ERR_NULL, "spec is NULL");
    ta_b200_sample_spec full;
    if (spec->struct_size == offsetof(ta_b200_sample_spec, torch_compat)) {      // the layout before torch_compat
        memset(&full, 0, sizeof(full));
        memcpy(&full, spec, offsetof(ta_b200_sample_spec, torch_compat));
        full.struct_size = sizeof(full);
        spec = &full;
    }
    if (spec->struct_size != sizeof(ta_b200_sample_spec))
        return ta::fail(TA_B200_ERR_SHAPE, "struct_size %u != %zu (ABI mismatch)", spec->struct_size, sizeof(ta_b200_sample_spec));
    if (spec->torch_compat) {
        int max_draw = -1;
        for (int j = 0; j < 13; ++j) {
            if (spec->draw[j] >= 13) return ta::fail(TA_B200_ERR_SHAPE, "draw[%d] = %d", j, (int)spec->draw[j]);
            if (spec->draw[j] > max_draw) max_draw = spec->draw[j];
        }
        if ((spec->draw[6] >= 0 || spec->draw[7] >= 0) && (spec->crop_h <= 0 || spec->crop_w <= 0))
            return ta::fail(TA_B200_ERR_SHAPE, "crop offsets are drawn but there is no crop size");
        const uint64_t off = spec->torch_state ? 0 : spec->torch_offset;
        if (off % 4 != 0) return ta::fail(TA_B200_ERR_UNSUPPORTED, "PyTorch generator offset %llu is not a multiple of 4", (unsigned long long)off);
    }
    if (spec->total < 0 || spec->frames < 1 || spec->first_sample < 0 ||
        (spec->first_sample == 0 && spec->total % spec->frames != 0))
        return ta::fail(TA_B200_ERR_SHAPE, "total = %d, frames = %d, first_sample = %d", spec->total, spec->frames, spec->first_sample);
    if (spec->img_h <= 0 || spec->img_w <= 0 || spec->crop_h < 0 || spec->crop_w < 0 || spec->crop_h > spec->img_h ||
        spec->crop_w > spec->img_w)
        return ta::fail(TA_B200_ERR_SHAPE, "image %dx%d, crop %dx%d", spec->img_h, spec->img_w, spec->crop_h, spec->crop_w);
    if (spec->factor_dtype != TA_B200_F32 && spec->factor_dtype != TA_B200_F16)
        return ta::fail(TA_B200_ERR_DTYPE, "factor_dtype %d", spec->factor_dtype);
    if (!spec->seed && !spec->torch_compat) return ta::fail(TA_B200_ERR_NULL, "seed is NULL");
    if (spec->total == 0) return TA_B200_OK;
    const int threads = 128, blocks = (spec->total + threads - 1) / threads;
    if (spec->factor_dtype == TA_B200_F32) ta::sample_params_kernel<float><<<blocks, threads, 0, (cudaStream_t)stream>>>(*spec);
    else ta::sample_params_kernel<__half><<<blocks, threads, 0, (cudaStream_t)stream>>>(*spec);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ta::cuda_fail(e, "launch(sample_params)");
    return TA_B200_OK;
}

int ta_b200_store_words(uint64_t *dst, uint64_t a, uint64_t b, void *stream)
{
    if (!dst) return ta::fail(TA_B200_ERR_NULL, "dst is NULL");
    ta::store_words_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(dst, a, b);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ta::cuda_fail(e, "launch(store_words)");
    return TA_B200_OK;
}

int ta_b200_debug_counters(uint64_t out[4], int reset)
{
    ta::DeviceState *s = nullptr;
    int rc = ta::current_device(&s, nullptr);
    if (rc != TA_B200_OK) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return ta::cuda_fail(e, "cudaDeviceSynchronize");
    if (out) {
        e = cudaMemcpy(out, s->counters, 4 * sizeof(uint64_t), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return ta::cuda_fail(e, "cudaMemcpy(counters)");
    }
    if (reset) {
        e = cudaMemset(s->counters, 0, 4 * sizeof(uint64_t));
        if (e != cudaSuccess) return ta::cuda_fail(e, "cudaMemset(counters)");
    }
    return TA_B200_OK;
}

// Same as ta_b200_fused_augment but with the staging assertions compiled in (apply must be 0).
int ta_b200_debug_fused_checked(const ta_b200_fused_params *p, void *stream)
{
    return ta::launch_fused(ta::Imported(p).ptr, (cudaStream_t)stream, true);
}

int ta_b200_debug_tile_footprint(int32_t interp, int32_t elem_bytes, int32_t h, int32_t w, int32_t oh, int32_t ow,
                                 float top, float left, int32_t flip, const float matrix[6], int32_t tile_x,
                                 int32_t tile_y, int32_t *row0, int32_t *xs, int32_t *xe, int32_t cap)
{
    ta::TileFootprint fp;
    const int chunk = 16 / (elem_bytes == 1 ? 1 : elem_bytes == 2 ? 2 : 4), pitch = ta::pitch_of(elem_bytes);
    const int mode = interp == TA_B200_BILINEAR ? 1 : 0;
    ta::tile_footprint(fp, mode, h, w, oh, ow, top, left, flip != 0, matrix, tile_x, tile_y);
    if (row0) *row0 = fp.row0;
    int group_xs[ta::kMaxRows / ta::kGroupRows];
    bool window = false;
    if (!ta::tile_plan(fp, mode, chunk, pitch, matrix, group_xs, &window)) return 0;
    for (int r = 0; r < fp.rows && r < cap; ++r) {
        xs[r] = group_xs[r / ta::kGroupRows];
        xe[r] = xs[r] + pitch;
    }
    return fp.rows;
}

int ta_b200_debug_crop_path(int32_t path)
{
    if (path < 0 || path > 2) return ta::fail(TA_B200_ERR_UNSUPPORTED, "crop path %d", path);
    ta::g_crop_path.store(path, std::memory_order_relaxed);
    return TA_B200_OK;
}

int ta_b200_debug_tile_height(int32_t rows)
{
    if (rows != 0 && rows != ta::kTileHShort && rows != ta::kTileH) return ta::fail(TA_B200_ERR_UNSUPPORTED, "tile height %d", rows);
    ta::g_tile_height.store(rows, std::memory_order_relaxed);
    return TA_B200_OK;
}

void ta_b200_debug_tile_shape(int32_t out[8])
{
    out[0] = ta::kTileW; out[1] = ta::kTileH; out[2] = ta::kMaxRows;
    out[3] = ta::pitch_of(4); out[4] = ta::pitch_of(2); out[5] = ta::pitch_of(1);
    out[6] = ta::kTileH; out[7] = ta::kMaxRows;      // (half pixels: the same shape as the others)
}

}  // extern "C"
