// What the kernels of the latent attention take (latent.cu, latent_mma.cu); the Python binding fills the same
// record (kernels._LatentArgs).
#pragma once
#include <cuda_runtime.h>

struct LatentArgs {
    // the step's rows
    const void* proj;            // [rows][ld_proj]: the low-rank query row (QR), the low-rank key/value row (KR + R), ...
    long long ld_proj;
    int q_off, kv_off;           // columns where the two begin
    void* cq;                    // [rows][QR]: the normed query latent, for the product that makes the heads' queries
    const float *wq_norm, *wkv_norm;   // [QR], [KR]
    const float* rate;           // [R / 2]: angle of pair i = position * rate[i] (0: the pair stays; times `mag` below)
    void* q;                     // [rows][H][D + R] the heads' queries as the product left them
    long long ldq;
    float* qa;                   // [rows][H][E], E = KR + R: per head the query against the latent, then its turned part
    long long ldqa;
    const void* gate;            // [rows][ld_gate], one logit per head (null: no gate)
    long long ld_gate;
    float* out;                  // [rows][H][KR]: sum of the weights times the latents, times sigmoid(gate)
    long long ldo;
    // geometry
    int H, D, R, KR, QR, E, EC;  // EC: a cache entry's size (the latent, the turned key part, zeros up to a multiple of 8)
    float eps, scale;
    long long rows;
    // the step and the cache
    const int *tok_pos, *tok_seq, *seq_start, *seq_pos0, *seq_end, *seq_slot;
    void* pool;                  // [pages][PAGE_TOKENS][EC]
    const int* ptab;             // [slots][ptab_stride]
    long long ptab_stride;
    int B, max_len;              // sequences; the longest run of new rows (the grid's bound)
    int splits, chunk;           // keys [s * chunk, (s + 1) * chunk) belong to split s; splits == 1: one block walks them all
    float* parts;                // splits > 1: [rows * H][splits][2 + KR] (maximum, sum, unnormalised output)
    // the prompt form that expands the latents into keys and values per head
    void* ckv;                   // [rows][EC] (or null): the step's cache entries once more, side by side, for a product
    const void* kvu;             // [rows][ld_kvu]: per head the unturned key (H * D), then per head the value (H * DV)
    long long ld_kvu;
    void* qkv;                   // [rows][ld_qkv]: queries, keys and values in heads of HD channels, zeros behind each head
    long long ld_qkv;
    int HD, DV;
    float mag;                   // the factor on every sine and cosine (1: a plain rotation)
    int no_entry;                // latent_prepare: the layer reads another layer's entries; only the query latent is made
};

// The splits' (maximum, sum, sums over the latents) of every (row, head) merged, normalised and gated (latent.cu); both
// forms of the attention end with it.
int cm_latent_attn_merge(int dt, const LatentArgs* args, cudaStream_t st);
