/* A C caller of the drop-in boundary, the way the reference's format layer would use it (format.m:343-363, 458-590,
 * 240-303): open a GGUF file, put its image on the device, build the tensor cache, run format_dispatch_matvec on one
 * layer's dense FFN and the lm_head + arg-max, and write the results for the test to compare.
 *
 *   format_client <model.gguf> <x.f32> <out.bin> <hidden> <ffn> <vocab>
 *
 * out.bin: act[ffn] floats, down[hidden] floats, logits[vocab] floats, token (uint32).
 * Uses only include/orome_cuda.h and include/orome_gguf.h (no CUDA headers): device buffers come from
 * orome_cuda_upload, results come back with orome_cuda_download. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "orome_cuda.h"
#include "orome_gguf.h"

#define CHECK(call)                                                                      \
    do {                                                                                 \
        int rc_ = (call);                                                                \
        if (rc_ != OROME_OK) {                                                           \
            fprintf(stderr, "%s: [%d] %s\n", #call, rc_, orome_cuda_last_error());       \
            return 2;                                                                    \
        }                                                                                \
    } while (0)

static void *device_floats(orome_cuda_ctx *ctx, const float *host, size_t n)
{
    void *dev = NULL;
    float *zero = host ? NULL : calloc(n, sizeof(float));
    if (orome_cuda_upload(ctx, host ? host : zero, n * sizeof(float), &dev) != OROME_OK) dev = NULL;
    free(zero);
    return dev;
}

int main(int argc, char **argv)
{
    if (argc != 7) { fprintf(stderr, "usage: %s model.gguf x.f32 out.bin hidden ffn vocab\n", argv[0]); return 1; }
    const int H = atoi(argv[4]), M = atoi(argv[5]), V = atoi(argv[6]);

    OromeGGUFFile *gf = orome_gguf_open(argv[1]);
    if (!gf) { fprintf(stderr, "gguf_open: %s\n", orome_cuda_last_error()); return 2; }
    const OromeGGUFMeta *meta = orome_gguf_meta(gf);
    if (meta->hidden_dim != H || meta->moe_intermediate != M || meta->vocab_size != V || meta->ffn_is_moe) {
        fprintf(stderr, "metadata mismatch: hidden %d ffn %d vocab %d moe %d\n", meta->hidden_dim, meta->moe_intermediate,
                meta->vocab_size, meta->ffn_is_moe);
        return 3;
    }

    orome_cuda_ctx *ctx = NULL;
    CHECK(orome_cuda_ctx_create(0, &ctx));
    OromeFormatProvider fp;
    CHECK(orome_format_provider_open_gguf(ctx, gf, &fp));

    OromeModelShape shape;
    memset(&shape, 0, sizeof shape);
    shape.num_layers = meta->num_layers; shape.hidden_dim = H; shape.moe_intermediate = M; shape.vocab_size = V;
    shape.num_attn_heads = meta->num_attn_heads; shape.num_kv_heads = meta->num_kv_heads; shape.head_dim = meta->attn_key_length;
    OromeLayerTensorCache *layers = calloc((size_t)meta->num_layers, sizeof *layers);
    OromeGlobalTensorCache globals;
    CHECK(orome_build_tensor_cache_gguf(&fp, &shape, OROME_VARIANT_DEFAULT, layers, &globals));

    float *x = malloc((size_t)H * sizeof(float));
    FILE *f = fopen(argv[2], "rb");
    if (!f || fread(x, sizeof(float), (size_t)H, f) != (size_t)H) { fprintf(stderr, "cannot read %s\n", argv[2]); return 4; }
    fclose(f);

    void *x_dev = device_floats(ctx, x, (size_t)H), *act_dev = device_floats(ctx, NULL, (size_t)M);
    void *down_dev = device_floats(ctx, NULL, (size_t)H), *logits_dev = device_floats(ctx, NULL, (size_t)V);
    void *token_dev = device_floats(ctx, NULL, 1);
    if (!x_dev || !act_dev || !down_dev || !logits_dev || !token_dev) { fprintf(stderr, "%s\n", orome_cuda_last_error()); return 5; }

    /* encode_dense_ffn (engine.m:342-392), then the lm_head on the FFN output and the arg-max of the logits */
    CHECK(orome_cuda_gate_up_swiglu(ctx, &layers[0].dense_gate, &layers[0].dense_up, x_dev, act_dev, 1, 0, 0, NULL));
    CHECK(orome_format_dispatch_matvec(ctx, &layers[0].dense_down, act_dev, 0, down_dev, 0, NULL));
    CHECK(orome_format_dispatch_matvec(ctx, &globals.lm_head, down_dev, 0, logits_dev, 0, NULL));
    CHECK(orome_cuda_argmax(ctx, logits_dev, (uint32_t)V, token_dev, NULL));
    int status = 0;
    CHECK(orome_cuda_status(ctx, &status));

    /* results back to the host (the reference reads its shared buffers in place, engine.m:1057) */
    f = fopen(argv[3], "wb");
    if (!f) return 6;
    float *host = malloc((size_t)(M + H + V + 1) * sizeof(float));
    CHECK(orome_cuda_download(ctx, act_dev, host, (size_t)M * sizeof(float)));
    CHECK(orome_cuda_download(ctx, down_dev, host + M, (size_t)H * sizeof(float)));
    CHECK(orome_cuda_download(ctx, logits_dev, host + M + H, (size_t)V * sizeof(float)));
    CHECK(orome_cuda_download(ctx, token_dev, host + M + H + V, sizeof(uint32_t)));
    fwrite(host, sizeof(float), (size_t)(M + H + V + 1), f);
    fclose(f);

    orome_cuda_free(ctx, x_dev); orome_cuda_free(ctx, act_dev); orome_cuda_free(ctx, down_dev);
    orome_cuda_free(ctx, logits_dev); orome_cuda_free(ctx, token_dev);
    orome_free_tensor_cache(&fp, layers, meta->num_layers);
    orome_format_provider_close(&fp);
    orome_cuda_ctx_destroy(ctx);
    orome_gguf_close(gf);
    free(layers); free(x); free(host);
    return 0;
}
