/*
 * ta_b200.h - C ABI of the B200 (sm_100a) fused image-augmentation library.
 *
 * The reference project (yuhezhang-ai/triton-augment v0.3.0) has no FFI layer:
 * its seam is a Python call that launches a Triton kernel.  This header is the
 * same seam as a C ABI.  Each entry point names the reference interface it
 * replaces (paths relative to the reference project's root).
 *
 * Conventions
 *   - Every function returns TA_B200_OK (0) or a negative ta_b200_status_code.  Nothing
 *     throws, exits, or synchronises the device unless the comment says so.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *     Work is enqueued on it and the call returns immediately.
 *   - The caller owns every buffer.  Images are contiguous NCHW.  Device pointers
 *     must belong to the device that is current when the call is made.
 *   - Calls may be made concurrently from several host threads as long as their
 *     output buffers do not overlap.
 */
#ifndef TA_B200_H
#define TA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TA_B200_ABI_VERSION 1

typedef enum ta_b200_status_code {
    TA_B200_OK = 0,
    TA_B200_ERR_NULL = -1,         /* a required pointer is NULL */
    TA_B200_ERR_SHAPE = -2,        /* sizes not positive, or channels not in {1, 3} */
    TA_B200_ERR_DTYPE = -3,        /* dtype is none of the TA_B200_F32 ... TA_B200_U8_F16 codes */
    TA_B200_ERR_UNSUPPORTED = -4,  /* e.g. saturation/grayscale on 1-channel images */
    TA_B200_ERR_CUDA = -5,         /* a CUDA runtime call failed; see ta_b200_last_error() */
    TA_B200_ERR_SCRATCH = -6,      /* scratch buffer missing or too small */
    TA_B200_ERR_DEVICE = -7,       /* current device is not compute capability 10.x */
    TA_B200_ERR_TOO_LARGE = -8,    /* a size exceeds what the entry point supports */
    TA_B200_ERR_TIMEOUT = -9       /* a kernel gave up a bounded wait: see ta_b200_status() */
} ta_b200_status_code;

/* TA_B200_U8: `in` holds bytes, `out` and the factor vectors are float32; a byte b enters the
 * pipeline as b / 255 (torchvision's ToTensor scaling), so the result equals the float32 call on
 * in.float() / 255 within the float32 tolerance.  No counterpart in the reference, which takes
 * float tensors only; it saves three quarters of the input traffic.  Its grayscale-mean
 * pre-pass (TA_B200_CONTRAST_MEAN) needs rows of whole 16-byte units.
 * TA_B200_U8_F16: bytes in, `out` and the factor vectors float16; b / 255 is rounded to half
 * and the pixel then takes the float16 path (result within the float16 tolerance of the
 * float16 call on (in.float() / 255).half()).  TA_B200_CONTRAST_MEAN is not available. */
enum { TA_B200_F32 = 0, TA_B200_F16 = 1, TA_B200_U8 = 2, TA_B200_U8_F16 = 3 };
enum { TA_B200_NEAREST = 0, TA_B200_BILINEAR = 1 };
enum { TA_B200_CONTRAST_FAST = 0, TA_B200_CONTRAST_MEAN = 1 };

/* Which colour operations are compiled in.  The reference derives these from the
 * parameter VALUES (triton_augment/functional.py:1341-1344, 1356): an operation
 * is skipped only when its factor is exactly 1.0 for every image (mask all-false,
 * mean/std None).  An enabled operation clamps to [0, 1] even for images whose
 * factor is 1.0, so the caller must make the same decision to get the same
 * output for pixels outside [0, 1]. */
enum {
    TA_B200_APPLY_BRIGHTNESS = 1u << 0,
    TA_B200_APPLY_CONTRAST   = 1u << 1,
    TA_B200_APPLY_SATURATION = 1u << 2,
    TA_B200_APPLY_GRAYSCALE  = 1u << 3,
    TA_B200_APPLY_NORMALIZE  = 1u << 4
};

/*
 * Arguments of one fused pass.  Field for field this is the 27-argument kernel
 * launch at triton_augment/functional.py:1399-1431 (kernel signature
 * triton_augment/kernels/fused_kernel.py:60-98); mean/std travel by value
 * instead of as 3-element device tensors.
 */
typedef struct ta_b200_fused_params {
    uint32_t struct_size;     /* sizeof(ta_b200_fused_params), for ABI checking */
    int32_t  dtype;           /* TA_B200_F32 / TA_B200_F16: type of in, out and the factor vectors; TA_B200_U8, TA_B200_U8_F16 see above */
    int32_t  n, c, h, w;      /* input  [n, c, h, w]; c in {1, 3} */
    int32_t  oh, ow;          /* output [n, c, oh, ow] (the crop size) */
    const void *in;
    void       *out;
    const float   *top;       /* [n] crop offsets held as fp32, NULL = 0 */
    const float   *left;      /* [n], NULL = 0 */
    const uint8_t *flip;      /* [n] 0/1, NULL = no flip */
    const float   *matrix;    /* [n, 6] inverse affine rows (a b c d e f), NULL = crop/flip only
                                 (has_affine=False in the reference) */
    float    fill;            /* value of texels outside the image (affine only) */
    int32_t  interp;          /* TA_B200_NEAREST / TA_B200_BILINEAR (affine only) */
    uint32_t apply;           /* TA_B200_APPLY_* bits */
    const void    *brightness; /* [n] image dtype; may be NULL when its bit is clear */
    const void    *contrast;   /* [n] */
    const void    *saturation; /* [n] */
    const uint8_t *gray;       /* [n] 0/1 */
    float    mean[3];         /* already rounded to the image dtype by the caller */
    float    std[3];          /* (triton_augment/functional.py:1350-1351) */
    int32_t  contrast_mode;   /* FAST: (x-0.5)*f+0.5, the reference's fused behaviour
                                 (fused_kernel.py:245-250).  MEAN: x*f+mean_n*(1-f), the
                                 torchvision-exact formula of its stand-alone contrast kernel
                                 (kernels/color_normalize_kernel.py:37-77); needs gray_mean. */
    const float   *gray_mean; /* [n] per-image means written by ta_b200_gray_mean() */
    /* -- fields below exist when struct_size == sizeof(ta_b200_fused_params); a caller built against
     *    the layout that ended at gray_mean passes that smaller struct_size and they are not read -- */
    float    fill_rgb[3];     /* with fill_per_channel != 0: value of out-of-image texels per channel
                                 (torchvision's fill=[r, g, b]; the reference takes fill[0] for all
                                 channels, triton_augment/functional.py:942-945, and notes per-channel
                                 values as to do); 1-channel images use fill_rgb[0] */
    uint32_t fill_per_channel;
} ta_b200_fused_params;

/* ABI version of the loaded library (TA_B200_ABI_VERSION it was built with). */
int ta_b200_abi_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char *ta_b200_last_error(void);

/*
 * Did a kernel of this library give up on the current device?  The staged kernels wait on
 * shared-memory barriers with a time limit (2 s); a wait that runs out makes its thread block
 * stop, leave the rest of its tiles unwritten and raise a flag in host-visible memory.  The
 * launch itself has long returned TA_B200_OK by then, so the condition is reported here and by
 * the NEXT call of ta_b200_fused_augment(), ta_b200_fused_augment_at(), ta_b200_gray_mean() on
 * the device, and by ta_b200_fused_augment_host() at its final synchronisation: they return
 * TA_B200_ERR_TIMEOUT and enqueue nothing until the flag is acknowledged.  Reading the flag
 * does not synchronise anything; call this after your own stream synchronisation to learn
 * whether the outputs produced since the last check are complete.
 * acknowledge != 0 clears the flag.  Returns TA_B200_OK or TA_B200_ERR_TIMEOUT.
 * No counterpart in the reference (a Triton launch has no waits of its own).
 */
int ta_b200_status(int acknowledge);

/*
 * The fused pass on device buffers: inverse-affine / crop / flip gather with
 * nearest or bilinear sampling, then brightness, contrast, saturation,
 * per-image grayscale and normalize, one read of the source footprint and one
 * write of the output.
 * Replaces: the launch of fused_augment_kernel, triton_augment/functional.py:1399-1431
 * (kernel: triton_augment/kernels/fused_kernel.py:55-376 with the helpers of
 * triton_augment/kernels/geometric_kernel.py:178-283, 349-420).  With no-op arguments
 * it also replaces the stand-alone kernels launched at functional.py:254, 318, 462,
 * 530, 591, 675, 809 and 960.
 */
int ta_b200_fused_augment(const ta_b200_fused_params *p, void *stream);

/*
 * The same for a piece of a larger batch (a shard, a slice): first_image is the index of p's
 * first image within that batch.  The reference's compiled kernel evaluates the source x
 * coordinate of some pixels in a second operation order that depends on the pixel's linear
 * index in the launch (bilinear float32 outputs whose height and width are both not multiples of
 * 16); with first_image the pieces reproduce one reference launch over the whole batch bit for
 * bit.  ta_b200_fused_augment() is first_image = 0.  No counterpart in the reference.
 */
int ta_b200_fused_augment_at(const ta_b200_fused_params *p, uint32_t first_image, void *stream);

/*
 * Per-image mean of the grayscale of the image that contrast would see in a
 * sequential pipeline: geometry (as described by *p) followed by brightness (if
 * its bit is set).  Writes mean_out[n] (device, fp32 holding image-dtype-rounded
 * values).  `scratch` is device memory of at least ta_b200_gray_mean_scratch_bytes(p)
 * bytes, 256-byte aligned; it needs no initialisation and may be reused by the next
 * call on the same stream.  (That size includes room for the faster of the two kernels that
 * implement the pass; with less, but at least round_up(4 n, 256) + 4 n min(128, ceil(oh ow /
 * 4096)) bytes, the slower one runs.  Both are deterministic; they differ in the last bits.)
 * Replaces: rgb_to_grayscale + torch.mean + cast, triton_augment/functional.py:366-376.
 */
int ta_b200_gray_mean(const ta_b200_fused_params *p, float *mean_out,
                      void *scratch, size_t scratch_bytes, void *stream);
size_t ta_b200_gray_mean_scratch_bytes(const ta_b200_fused_params *p);

/*
 * Mean-mode contrast (TA_B200_CONTRAST_MEAN) in one call: the grayscale-mean reduction of
 * ta_b200_gray_mean() and the fused pass of ta_b200_fused_augment(), p->gray_mean not needed.
 * Writes the means to mean_out[n] (device) on the way.  The result is bit-identical to
 * ta_b200_gray_mean() followed by ta_b200_fused_augment().
 * By default the call makes those two launches.  After ta_b200_mean_path(1) (or 2), float32
 * images whose rows the staged kernels can read (16-byte aligned rows, see ta_b200_gray_mean) run
 * both as ONE cooperative launch instead: every thread block alternates between reduction tiles of
 * one image and fused-pass tiles of the image one (two) before it, so the second read of the source
 * comes from the L2 cache and there is no launch in between; a block that needs a mean which is not
 * final yet waits for it (bounded, see ta_b200_status()).  Same bits; on a B200 it measured slower
 * than two launches on large batches (both passes are bound by instruction issue, not by HBM),
 * which is why it is not the default.
 * `scratch`: device memory, 256-byte aligned, ta_b200_fused_augment_mean_scratch_bytes(p) bytes,
 * no initialisation needed, reusable by the next call on the same stream.
 * Replaces: adjust_contrast's three passes inside a composed pipeline,
 * triton_augment/functional.py:329-403 (the reference's fused kernel has the fast formula only).
 */
int ta_b200_fused_augment_mean(const ta_b200_fused_params *p, float *mean_out, void *scratch,
                               size_t scratch_bytes, void *stream);
size_t ta_b200_fused_augment_mean_scratch_bytes(const ta_b200_fused_params *p);

/*
 * ta_b200_gray_mean() for callers that cannot allocate device memory.  (No counterpart in
 * the reference, which allocates freely through torch.)
 *
 * Some users of this library are handed their device memory once and may not ask for more:
 * a plugin inside a host application that owns the CUDA allocator, a data-loading service
 * whose memory budget is frozen after start-up, code that runs where a cudaMalloc would
 * stall or is forbidden.  For them the scratch lives inside the library, in a fixed 1 MiB
 * array of device memory that every GPU using the library holds from load to process exit.
 * The call itself allocates nothing and frees nothing, on the host's CUDA heap or through
 * any library (the very first launch of a kernel on a device may still make the CUDA runtime
 * load that kernel's code, so count on "allocates nothing" from the second call on); the
 * caller still supplies the input image, the parameter vectors and mean_out[n], exactly as
 * for ta_b200_gray_mean() - p->out may be NULL, the pre-pass writes no image.
 * This entry always runs the gather kernel (the slower of the two that ta_b200_gray_mean()
 * chooses from): the faster one needs megabytes of partial sums, more than the fixed array.
 *
 * Limit: counters plus partial sums must fit the array, i.e.
 *     round_up(4 n, 256) + 4 n min(128, ceil(oh ow / 4096))  <=  1 048 576 bytes
 * (for example about 18 700 images of 224x224, or 2032 images of 1024x1024).  A larger call is
 * refused with TA_B200_ERR_TOO_LARGE and a message saying how much was needed; split the
 * batch or use ta_b200_gray_mean() with your own scratch.
 *
 * The first call on each device looks up the array's device address (one runtime query,
 * made with that device current).  Make that first call before starting any stream capture.
 * All calls on a device share the one array and it keeps what the last call left in it: the
 * part that must start at zero is cleared on `stream` at the start of every call, and two
 * calls whose kernels can overlap on the GPU (different streams, no ordering between them)
 * race on it and produce garbage - order them yourself.
 */
int ta_b200_gray_mean_static(const ta_b200_fused_params *p, float *mean_out, void *stream);

/*
 * Host-buffer variant of ta_b200_fused_augment(): p->in and p->out are HOST
 * pointers (pinned memory gives full PCIe speed); every per-image vector and the
 * matrix are host pointers too.  The batch is cut into slices that flow through
 * upload -> kernel -> download on three streams, so copies overlap the kernel.
 * Device staging buffers are allocated on first use and cached per device.
 * Of image planes of 1 MiB or more only the box of source pixels that the call
 * reads (known from top / left / matrix and the output size) is uploaded, when
 * that is cheaper than copying whole slices (priced from measured copy rates).
 * Synchronous: returns when p->out is complete.
 * Replaces: the host-tensor path of the transform classes, which upload with
 * .cuda() before calling the kernel (triton_augment/transforms.py:1498-1504).
 */
int ta_b200_fused_augment_host(const ta_b200_fused_params *p);

/* Frees what ta_b200_fused_augment_host() keeps on the current device between calls (staging
 * buffers, three streams, events) after waiting for them; the next host call re-creates them. */
int ta_b200_host_release(void);

/*
 * Inverse affine matrices on the device in one launch: angle[n], translate[n,2],
 * scale[n], shear[n,2] (degrees / pixels, device fp32; center may be NULL = image
 * centre) -> matrix[n,6].  Same operation order as
 * triton_augment/functional.py:853-890 (_get_inverse_affine_matrix).
 */
int ta_b200_inverse_affine_matrix(int32_t n, const float *center, const float *angle,
                                  const float *translate, const float *scale,
                                  const float *shear, float *matrix, void *stream);

/*
 * All per-sample parameters of one TritonFusedAugment call in ONE launch: the random draws,
 * their broadcast over video frames, and the inverse affine matrices.  Replaces, as an opt-in,
 * the ~18 separate draws and elementwise operations of triton_augment/transforms.py:1431-1531
 * and functional.py:1308-1397.  The distributions are the reference's (uniform ranges, integer
 * crop offsets, Bernoulli masks); the random STREAM is not: values come from a Philox4x32-10
 * generator of this library keyed by *seed (device memory) and the parameter-set index, so a
 * seed does not reproduce the reference's parameters.  No counterpart in the reference.
 *
 * Sample i of `total` uses parameter set p(i): with frames == 1, p = same_on_batch ? 0 : i;
 * with frames = T > 1 (sample i = frame i % T of video i / T),
 * p = (same_on_batch ? 0 : i / T) * (same_on_frame ? 1 : T) + (same_on_frame ? 0 : i % T).
 * Every output pointer may be NULL (not written).  Factors are written in `factor_dtype`
 * (TA_B200_F32 or TA_B200_F16); a range with lo == hi is written as that constant.
 */
typedef struct ta_b200_sample_spec {
    uint32_t struct_size;       /* sizeof(ta_b200_sample_spec) */
    int32_t  total, frames;
    int32_t  same_on_batch, same_on_frame;
    int32_t  img_h, img_w;      /* input size: translation range and crop range */
    int32_t  crop_h, crop_w;    /* 0, 0: no crop (top = left = 0) */
    int32_t  factor_dtype;
    float    degrees[2];        /* angle ~ U(degrees[0], degrees[1]) */
    float    translate[2];      /* tx ~ U(-translate[0] * img_w, +...), ty likewise with img_h */
    float    scale[2];          /* scale ~ U */
    float    shear[4];          /* shear_x ~ U(shear[0], shear[1]), shear_y ~ U(shear[2], shear[3]) */
    float    flip_p, grayscale_p;
    float    brightness[2], contrast[2], saturation[2];
    const uint64_t *seed;       /* device: 64-bit seed of this call */
    float   *top, *left;        /* [total] */
    uint8_t *flip, *gray;       /* [total] */
    float   *matrix;            /* [total, 6] */
    void    *brightness_out, *contrast_out, *saturation_out;   /* [total] factor_dtype */
    float   *angle_out, *translate_out, *scale_out, *shear_out; /* [total], [total,2], [total], [total,2]: the draws behind matrix */
    /* -- fields below exist when struct_size == sizeof(ta_b200_sample_spec); the layout that ended at
     *    shear_out is still accepted (torch_compat reads as 0) -- */
    /*
     * torch_compat != 0: reproduce the parameters that the reference's own sequence of draws
     * (one `uniform_` / `randint` / `rand` call of [parameter sets] values per parameter,
     * triton_augment/transforms.py:1431-1481, 1712-1751, 637-668) takes from PyTorch's CUDA
     * generator, in this one launch.  PyTorch's generator is Philox4x32-10 keyed by its seed; a
     * draw of up to (SM count x resident threads) values gives value i the first output word of
     * counter (offset / 4, i) and advances the offset by 4.  draw[j] says which draw of the call
     * (0, 1, 2 ... in the reference's order) parameter j comes from, or -1 for a parameter the
     * configuration does not draw (it gets its neutral value: angle 0, translation 0, scale 1,
     * shear 0, offsets 0, no flip, factors 1, no grayscale).  j: 0 angle, 1 tx, 2 ty, 3 scale,
     * 4 shear x, 5 shear y, 6 top, 7 left, 8 flip, 9 brightness, 10 contrast, 11 saturation,
     * 12 grayscale.  In this mode translate[] holds the translation ranges in PIXELS (the reference
     * multiplies fraction and image size in double precision before the draw).  The generator's (seed, offset) at the start of the call come from
     * torch_state (device, two 64-bit words: a captured graph can be replayed with new values) or,
     * if that is NULL, from torch_seed / torch_offset.  The caller advances PyTorch's offset by
     * 4 x (number of draws) afterwards.  Bits of torch_compat above bit 0 select how two float
     * roundings are done, which is a property of the PyTorch build: bit 1 = the conversion of a
     * random word to (0, 1] is a fused multiply-add, bit 2 = `rand * range + from` is.  seed is
     * not read in this mode.
     */
    int32_t  torch_compat;
    int8_t   draw[13];
    int8_t   pad_[3];
    uint64_t torch_seed, torch_offset;
    const uint64_t *torch_state;
    int32_t  first_sample;      /* the launch covers samples first_sample .. first_sample + total - 1 of a larger
                                   batch (a shard): entry i of every output belongs to sample first_sample + i */
    int32_t  pad2_;
} ta_b200_sample_spec;

int ta_b200_sample_params(const ta_b200_sample_spec *spec, void *stream);

/* dst[0] = a, dst[1] = b on `stream` (device memory): how a caller refreshes the torch_state of a
 * captured ta_b200_sample_params launch before replaying the graph - the values travel as
 * kernel arguments, so no host buffer has to outlive the call. */
int ta_b200_store_words(uint64_t *dst, uint64_t a, uint64_t b, void *stream);

/*
 * Diagnostics.  ta_b200_debug_counters copies {tiles staged through shared memory,
 * tiles that took the direct-gather path, staging violations seen by a checked
 * build, barrier waits that ran out} accumulated on the current device since the
 * last reset into out[4] (synchronises the device).
 */
int ta_b200_debug_counters(uint64_t out[4], int reset);

/* ta_b200_fused_augment() with assertions on every shared-memory tap compiled in
 * (affine only, p->apply must be 0); violations show up in ta_b200_debug_counters()[2]. */
int ta_b200_debug_fused_checked(const ta_b200_fused_params *p, void *stream);

/*
 * Host-only helper for tests: the source rows and per-row column ranges that the
 * staged affine kernel would fetch for one output tile.  Returns the number of rows
 * (0 if the tile would not be staged), writes the first row to *row0 and per-row
 * [xs, xe) to xs[]/xe[] (capacity `cap` rows).
 */
int ta_b200_debug_tile_footprint(int32_t interp, int32_t elem_bytes, int32_t h, int32_t w,
                                 int32_t oh, int32_t ow, float top, float left, int32_t flip,
                                 const float matrix[6], int32_t tile_x, int32_t tile_y,
                                 int32_t *row0, int32_t *xs, int32_t *xe, int32_t cap);
/* Time limit of the kernels' barrier waits in nanoseconds (0 restores the default of 2 s), and the
 * number of one tile whose producer warp leaves without signalling the tile's barrier in the staged
 * kernels launched from now on (-1: none), process-wide.  With a small limit and a tile number a
 * test makes a wait run out on purpose - nothing faults, traps or spins without bound: the
 * thread block that owns the tile gives up after the limit, the launch completes, and
 * ta_b200_status() / ta_b200_debug_counters()[3] report it. */
int ta_b200_debug_wait(uint64_t limit_ns, int32_t skip_arrive_tile);
/* How ta_b200_fused_augment_mean() runs, process-wide: 0 = two launches (default), 1 / 2 = one
 * cooperative launch where the images allow it, the fused pass one / two images behind the
 * reduction.  Identical output. */
int ta_b200_mean_path(int32_t one_launch);
/* Which kernel runs calls without a matrix (crop / flip / colour), process-wide: 0 = chosen
 * by size (default: large fp32 batches go through the staged kernel, everything else through
 * the crop kernels), 1 = always the crop kernels, 2 = the staged kernel whenever the tensors
 * allow it.  Both produce identical output; the switch exists so that tests can compare them. */
int ta_b200_debug_crop_path(int32_t path);
/* Tile height of the staged kernel for float32 and float16 images, process-wide: 0 = chosen by
 * the call (default: 64 rows; 32 rows with a deeper ring for outputs of at most 256 rows
 * (float32) or 96 rows (float16) whose last row of 64-row tiles would be at most half full, and for
 * every float32 call without a matrix), 32 / 64 = that height for every call.  Identical output; the switch exists so that tests can
 * compare the shapes. */
int ta_b200_debug_tile_height(int32_t rows);
/* ta_b200_fused_augment_host(): 1 = upload only the box of each large image that the call reads
 * when the copy plan is cheaper than whole slices (default), 0 = upload every image whole, 2 =
 * boxes for every call on large images.  Identical output; for tests and measurements. */
int ta_b200_debug_host_upload(int32_t trimmed);
/* Tile shape of the staged affine kernel: out[0] = width, out[1] = height, out[2] = source-row
 * capacity, out[3], out[4], out[5] = staged row pitch in elements for 4-, 2- and 1-byte source
 * elements; out[6], out[7] repeat height and row capacity (half output pixels once had their own). */
void ta_b200_debug_tile_shape(int32_t out[8]);

#ifdef __cplusplus
}
#endif
#endif /* TA_B200_H */
