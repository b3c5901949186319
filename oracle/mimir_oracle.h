/* mimir_oracle.h — TEST INFRASTRUCTURE: prototypes of the plain-C restatement (mimir_oracle.c).
 * One sample per call; see the .c file for the reference file:line each function follows. */
#ifndef MIMIR_ORACLE_H
#define MIMIR_ORACLE_H
#ifdef __cplusplus
extern "C" {
#endif
void mo_linear(const float* x, const float* w, const float* bias, float* y, long rows, int in_f, int out_f);
void mo_matmul(const float* A, const float* B, float* C, long M, long K, long N);
void mo_attention(const float* x, const float* wqkv, const float* wout, float* y, int seq, int E, int heads, int causal);
void mo_conv2d(const float* x, const float* w, float* y, int ic, int oc, int h, int wd, int k, int stride, int pad, int relu);
void mo_layernorm(const float* x, const float* gamma, const float* beta, float* y, long rows, int n, float eps);
void mo_rmsnorm(const float* x, const float* gamma, long n_gamma, float* y, long n, float eps);
void mo_groupnorm(const float* x, const float* gamma, const float* beta, float* y, int C_, int h, int w, int G, float eps);
void mo_softmax(const float* x, float* y, long n, int log_softmax);
int  mo_eltwise(int op, const float* a, const float* b, float* y, long n, long nb);
void mo_embedding(const float* ids, const float* table, float* y, long n_ids, int vocab, int dim, int padding_idx);
void mo_upsample_nearest(const float* x, float* y, int ch, int in_h, int in_w, int sh, int sw);
void mo_permute(const float* x, float* y, int nd, const int* shape, const int* dims);
void mo_token_mean_pool(const float* x, float* y, int seq, int dim);
void mo_global_avgpool(const float* x, float* y, int ch, int h, int w);
void mo_leaky_relu(const float* a, float* y, long n, float alpha);
void mo_cross_attention(const float* q_in, const float* kv_in, const float* wq, const float* wkv, const float* wout, float* y,
                        int q_len, int kv_len, int E, int heads, int causal);
void mo_depthwise_conv2d(const float* x, const float* w, const float* bias, float* y, int ch, int h, int wd, int k, int stride,
                         int pad);
void mo_conv1d(const float* x, const float* w, const float* bias, float* y, int ic, int oc, int len, int k, int stride, int pad);
void mo_conv_transpose2d(const float* x, const float* w, float* y, int ic, int oc, int h, int wd, int k, int stride, int pad,
                         int relu);
void mo_pool2d(int is_max, const float* x, float* y, int ch, int h, int wd, int kh_n, int kw_n, int sh, int sw, int ph, int pw);
void mo_pad2d(int mode, const float* x, float* y, int ch, int h, int wd, int ph, int pw);
void mo_pixel_shuffle(const float* x, float* y, int ic, int h, int wd, int r);
void mo_upsample_bilinear(const float* x, float* y, int ch, int h, int wd, int oh, int ow, int half_pixel);
void mo_batch_matmul(const float* A, const float* B, float* C, long nb, int M, int K, int N);
void mo_batchnorm_inference(const float* x, const float* w, long n_w, float* y, long n, float eps);
void mo_batchnorm_running(const float* x, const float* gamma, const float* beta, const float* mean, const float* var,
                          float* y, int batch, int channels, long spatial, float eps);
void mo_attention_qkv(const float* q, const float* k, const float* v, float* y, int seq, int d_model, int heads);
void mo_instance_norm2d(const float* x, const float* w, float* y, int ch, int h, int wd, float eps);
long mo_embedding_bag(const float* ids, long n_ids, const float* offsets, long n_off, const float* table, float* y, int vocab,
                      int dim, int padding_idx);
void mo_patch_embed(const float* x, const float* w, float* y, int d_model, int seq_text, int num_patches, int patch_dim);
void mo_bilinear(const float* x1, const float* x2, const float* w, const float* bias, float* y, long rows, int in1, int in2,
                 int out_f);
void mo_maxpool1d(const float* x, float* y, int ch, long len, int k, int stride, int pad);
void mo_attention_core(const float* qkv, float* att, int seq, int E, int heads, int causal);
void mo_conv2d_dilated(const float* x, const float* w, const float* bias, float* y, int ic, int oc, int h, int wd, int k, int stride,
                       int pad, int dil, int avx2_lanes);
void mo_conv_transpose2d_scatter(const float* x, const float* w, const float* bias, float* y, int ic, int oc, int h, int wd, int k,
                                 int stride, int pad);
void mo_batchnorm_batchstats(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels, long spatial,
                             float eps);
void mo_elu(const float* a, float* y, long n, float alpha);
void mo_recurrent(int kind, const float* x, const float* w, float* y, int T, int I, int H, int use_bias);
#ifdef __cplusplus
}
#endif
#endif
