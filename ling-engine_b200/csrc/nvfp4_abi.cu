// nvfp4_abi.cu -- C-ABI entry points of the NVFP4 prefill-chunk path: the quantizers and GEMMs on host buffers (copy in,
// launch, copy out), as the reference's kernel tests drive them (tests/prefill_tests.cu in the reference project), and the
// chunk's feed-forward stack (norm -> gate|up with fused SwiGLU -> down into the residual, layer after layer) held on the
// device for the mixed prefill + decode pass, and one DeltaNet layer's mixer on the prefill path (norm -> in projections ->
// conv, gating, chunked delta rule -> gated norm -> out projection into the residual).
#include <cmath>
#include <cstring>
#include <memory>

#include "abi_util.h"
#include "gdn_chunk.h"
#include "nvfp4.h"

using namespace lb;

namespace {

bool multiple(int v, int m) { return v > 0 && v % m == 0; }

// An operand on the device built from host codes [rows][K/2] and row-major scales [rows][K/16].
int upload_operand(Scratch& sc, Fp4Operand& o, const uint8_t* q, const uint8_t* sf, int rows, int K) {
  o.rows = rows, o.K = K;
  o.codes = sc.put(q, size_t(rows) * (K / 2));
  o.sf = sc.get<uint8_t>(fp4_sf_bytes(rows, K));
  uint8_t* raw = sc.put(sf, size_t(rows) * (K / 16));
  LB_PTR(o.codes && o.sf && raw);
  LB_TRY(fp4_sf_tile_launch(raw, o.sf, rows, K, 0));
  return make_fp4_map(o);
}

int read_flag(const int* err, const char* what) {
  int code = 0;
  LB_CUDA(cudaMemcpy(&code, err, 4, cudaMemcpyDeviceToHost));
  if (code) {
    set_error(std::string(what) + ": device error word = " + std::to_string(code));
    return LING_B200_ERR_DEVICE_FLAG;
  }
  return LING_B200_OK;
}

}  // namespace

// A DeltaNet layer's mixer on the prefill path (Engine::forward's linear-attention branch over many rows, quantized path):
// one layer's weights and session state, and the activation buffers every layer shares.
struct GdnWeights {
  __nv_bfloat16 *norm = nullptr, *convw = nullptr, *wa = nullptr, *wb = nullptr, *A_log = nullptr, *dt_bias = nullptr, *lin_norm = nullptr;
  Fp4Operand in_qkv, in_z, out;
  float s_qkv = 1.f, s_z = 1.f, s_out = 1.f;
  float *state = nullptr, *conv = nullptr;  // [HV][128][128], [C][3]
};
struct GdnBuffers {
  int H = 0, Hk = 0, HV = 0, C = 0, Vs = 0, max_rows = 0;
  float eps = 1e-6f, in_scale = 16.f / (6.f * 448.f), mid_scale = 64.f / (6.f * 448.f);  // as the feed-forward stack's
  float *xn = nullptr, *pre = nullptr, *post = nullptr, *z = nullptr, *g = nullptr, *beta = nullptr, *core = nullptr;
  Fp4Operand x, mid;
  uint8_t* chunk_scratch = nullptr;  // gdn_chunk_scratch_bytes(max_rows, HV)
};

// The chunk's feed-forward stack: per layer the post-attention norm weight and the three NVFP4 matrices.
struct ling_b200_nvfp4_ffn {
  int device = 0, layers = 0, H = 0, I = 0, max_rows = 0;
  int ctas = 0;  // CTAs of each GEMM launch (0: one per SM)
  float eps = 1e-6f;
  struct Layer {
    __nv_bfloat16* norm = nullptr;
    Fp4Operand gate, up, down;
    float in_scale = 1.f, mid_scale = 1.f;  // the activations' static input scales
    float s_gate = 1.f, s_up = 1.f, s_down = 1.f;  // the weights' tensor scales
  };
  std::vector<Layer> L;
  GdnBuffers mix;                // with mixers (ling_b200_nvfp4_ffn_add_mixers): the DeltaNet layers' mixer runs before their FFN
  std::vector<GdnWeights> mixers;  // by layer; a full-attention layer's entry stays empty
  // with a verify context attached (ling_b200_nvfp4_ffn_attach_context): the full-attention layers' mixer runs through that
  // context's own FP8 projections and attention kernels, on the chunk session's pages
  ling_b200_ctx* attn_ctx = nullptr;
  int attn_slot = 0, attn_pos0 = 0, attn_every = 0;
  float* h = nullptr;      // residual [max_rows][H]
  Fp4Operand x, mid;       // the two GEMMs' activations
  int* err = nullptr;
  float* pin_in = nullptr;   // pinned host staging for the end-to-end call
  float* pin_out = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  Scratch mem;
  ~ling_b200_nvfp4_ffn() {
    if (pin_in) cudaFreeHost(pin_in);
    if (pin_out) cudaFreeHost(pin_out);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (stream) cudaStreamDestroy(stream);
  }
};

namespace {

int alloc_operand(Scratch& sc, Fp4Operand& o, int rows, int K) {
  o.rows = rows, o.K = K;
  o.codes = sc.get<uint8_t>(size_t(rows) * (K / 2));
  o.sf = sc.get<uint8_t>(fp4_sf_bytes(rows, K));
  LB_PTR(o.codes && o.sf);
  return make_fp4_map(o);
}

// One synthetic NVFP4 matrix: BF16 N(0, 0.02) from the library's generator, rounded as a checkpoint's NVFP4 is.
int synth_matrix(ling_b200_nvfp4_ffn* f, Fp4Operand& o, int N, int K, uint64_t key, __nv_bfloat16* tmp, unsigned* amax, float* scale2_dev,
                 float* scale2) {
  LB_TRY(alloc_operand(f->mem, o, N, K));
  LB_TRY(fill_bf16_launch(nullptr, key, 0.02f, 0.f, 1, tmp, size_t(N) * K, f->stream));
  LB_CUDA(cudaMemsetAsync(amax, 0, 4, f->stream));
  LB_TRY(fp4_quant_weight_launch(tmp, N, K, o.codes, o.sf, true, scale2_dev, amax, f->stream));
  LB_CUDA(cudaMemcpyAsync(scale2, scale2_dev, 4, cudaMemcpyDeviceToHost, f->stream));
  LB_CUDA(cudaStreamSynchronize(f->stream));
  return LING_B200_OK;
}

bool gdn_shape_ok(int hidden, int k_heads, int v_heads) {
  return multiple(hidden, 256) && k_heads >= 1 && v_heads >= 1 && v_heads % k_heads == 0 && multiple(v_heads * 128, 256) &&
         multiple((2 * k_heads + v_heads) * 128, 256);
}

int synth_operand(Scratch& mem, cudaStream_t st, Fp4Operand& o, int N, int K, uint64_t key, __nv_bfloat16* tmp, unsigned* amax, float* scale2_dev,
                  float* scale2) {
  LB_TRY(alloc_operand(mem, o, N, K));
  LB_TRY(fill_bf16_launch(nullptr, key, 0.02f, 0.f, 1, tmp, size_t(N) * K, st));
  LB_CUDA(cudaMemsetAsync(amax, 0, 4, st));
  LB_TRY(fp4_quant_weight_launch(tmp, N, K, o.codes, o.sf, true, scale2_dev, amax, st));
  LB_CUDA(cudaMemcpyAsync(scale2, scale2_dev, 4, cudaMemcpyDeviceToHost, st));
  LB_CUDA(cudaStreamSynchronize(st));
  return LING_B200_OK;
}

int gdn_buffers_create(Scratch& m, int hidden, int k_heads, int v_heads, int max_rows, GdnBuffers& b) {
  b.H = hidden, b.Hk = k_heads, b.HV = v_heads, b.max_rows = max_rows;
  b.C = (2 * k_heads + v_heads) * 128, b.Vs = v_heads * 128;
  const size_t R = size_t(max_rows);
  b.xn = m.get<float>(R * hidden), b.pre = m.get<float>(R * b.C), b.post = m.get<float>(R * b.C);
  b.z = m.get<float>(R * b.Vs), b.g = m.get<float>(R * v_heads), b.beta = m.get<float>(R * v_heads), b.core = m.get<float>(R * b.Vs);
  b.chunk_scratch = m.get<uint8_t>(gdn_chunk_scratch_bytes(max_rows, v_heads), false);
  LB_PTR(b.xn && b.pre && b.post && b.z && b.g && b.beta && b.core && b.chunk_scratch);
  LB_TRY(alloc_operand(m, b.x, max_rows, hidden));
  return alloc_operand(m, b.mid, max_rows, b.Vs);
}

// One layer's synthetic weights (the library's generator under the layer's tensor streams) and a zero state.
int gdn_weights_create(Scratch& m, cudaStream_t st, const GdnBuffers& b, int layer, uint64_t seed, __nv_bfloat16* wtmp, unsigned* amax, float* s2,
                       GdnWeights& w) {
  const int H = b.H, HV = b.HV;
  w.norm = m.get<__nv_bfloat16>(H), w.convw = m.get<__nv_bfloat16>(size_t(b.C) * 4);
  w.wa = m.get<__nv_bfloat16>(size_t(HV) * H), w.wb = m.get<__nv_bfloat16>(size_t(HV) * H);
  w.A_log = m.get<__nv_bfloat16>(HV), w.dt_bias = m.get<__nv_bfloat16>(HV), w.lin_norm = m.get<__nv_bfloat16>(128);
  w.state = m.get<float>(size_t(HV) * 128 * 128), w.conv = m.get<float>(size_t(b.C) * 3);
  LB_PTR(w.norm && w.convw && w.wa && w.wb && w.A_log && w.dt_bias && w.lin_norm && w.state && w.conv);
  auto key = [&](int t) { return stream_key(seed, weight_stream(layer, t)); };
  LB_TRY(fill_bf16_launch(nullptr, key(LING_B200_T_INPUT_NORM), 0.02f, 0.f, 1, w.norm, H, st));
  LB_TRY(fill_bf16_launch(nullptr, key(LING_B200_T_CONV), 0.3f, 0.f, 1, w.convw, size_t(b.C) * 4, st));
  LB_TRY(fill_bf16_launch(nullptr, key(LING_B200_T_IN_A), 0.02f, 0.f, 1, w.wa, size_t(HV) * H, st));
  LB_TRY(fill_bf16_launch(nullptr, key(LING_B200_T_IN_B), 0.02f, 0.f, 1, w.wb, size_t(HV) * H, st));
  LB_TRY(fill_bf16_launch(nullptr, key(LING_B200_T_A_LOG), 0.5f, -1.f, 1, w.A_log, HV, st));
  LB_TRY(fill_bf16_launch(nullptr, key(LING_B200_T_DT_BIAS), 0.5f, 0.f, 1, w.dt_bias, HV, st));
  LB_TRY(fill_bf16_launch(nullptr, key(LING_B200_T_LIN_NORM), 0.1f, 1.f, 1, w.lin_norm, 128, st));
  LB_TRY(synth_operand(m, st, w.in_qkv, b.C, H, key(LING_B200_T_IN_QKV), wtmp, amax, s2, &w.s_qkv));
  LB_TRY(synth_operand(m, st, w.in_z, b.Vs, H, key(LING_B200_T_IN_Z), wtmp, amax, s2, &w.s_z));
  return synth_operand(m, st, w.out, H, b.Vs, key(LING_B200_T_OUT), wtmp, amax, s2, &w.s_out);
}

// h [rows][H] += out( gated_norm( delta_rule( conv(in_qkv(norm(h))), gating(in_a, in_b) ), in_z(norm(h)) ) ); the layer's state and
// window advance.  Ten launches on `st`.
int gdn_mixer_run(GdnBuffers& b, const GdnWeights& w, float* h, int rows, int* err, int ctas, cudaStream_t st) {
  b.x.rows = rows, b.mid.rows = rows;
  LB_TRY(make_fp4_map(b.x));
  LB_TRY(make_fp4_map(b.mid));
  LB_TRY(fp4_rmsnorm_quant_launch(h, w.norm, b.xn, rows, b.H, b.eps, 1.f / b.in_scale, b.x.codes, b.x.sf, true, st));
  Fp4GemmCall a;
  a.X = &b.x, a.W = &w.in_qkv, a.alpha = b.in_scale * w.s_qkv, a.y = b.pre, a.ldy = b.C, a.err_flag = err, a.ctas = ctas;
  LB_TRY(fp4_gemm_launch(a, st));
  Fp4GemmCall zc;
  zc.X = &b.x, zc.W = &w.in_z, zc.alpha = b.in_scale * w.s_z, zc.y = b.z, zc.ldy = b.Vs, zc.err_flag = err, zc.ctas = ctas;
  LB_TRY(fp4_gemm_launch(zc, st));
  if (b.H % 128 == 0) LB_TRY(ab_gating_mma_launch(b.xn, w.wa, w.wb, w.A_log, w.dt_bias, b.g, b.beta, rows, b.H, b.HV, st));
  else LB_TRY(ab_gating_rows_launch(b.xn, w.wa, w.wb, w.A_log, w.dt_bias, b.g, b.beta, rows, b.H, b.HV, st));
  LB_TRY(conv_rows_launch(b.pre, w.convw, w.conv, rows, b.C, b.post, st));
  LB_TRY(gdn_chunk_launch(b.post, b.g, b.beta, rows, b.Hk, b.HV, 128, 128, w.state, b.core, b.chunk_scratch, st));
  LB_TRY(fp4_gated_norm_quant_launch(b.core, b.z, w.lin_norm, rows, b.Vs, b.eps, 1.f / b.mid_scale, b.mid.codes, b.mid.sf, true, st));
  Fp4GemmCall o;
  o.X = &b.mid, o.W = &w.out, o.alpha = b.mid_scale * w.s_out, o.y = h, o.ldy = b.H, o.accumulate = true, o.err_flag = err, o.ctas = ctas;
  return fp4_gemm_launch(o, st);
}

// The stack over rows [0, rows) of the residual, on the object's stream.
int ffn_run(ling_b200_nvfp4_ffn* f, int rows) {
  f->x.rows = rows, f->mid.rows = rows;
  LB_TRY(make_fp4_map(f->x));
  LB_TRY(make_fp4_map(f->mid));
  for (size_t l = 0; l < f->L.size(); ++l) {
    const auto& L = f->L[l];
    if (l < f->mixers.size() && f->mixers[l].in_qkv.codes) LB_TRY(gdn_mixer_run(f->mix, f->mixers[l], f->h, rows, f->err, f->ctas, f->stream));
    if (f->attn_ctx && f->attn_every > 0 && int(l) % f->attn_every == f->attn_every - 1) {
      // the attention layer works on the context's stream and returns when it is complete; what this stream has queued
      // on the residual comes first
      LB_CUDA(cudaStreamSynchronize(f->stream));
      LB_TRY(ling_b200_chunk_attention_layer(f->attn_ctx, f->attn_slot, int(l), f->attn_pos0, rows, f->h));
      LB_CUDA(cudaSetDevice(f->device));
    }
    LB_TRY(fp4_rmsnorm_quant_launch(f->h, L.norm, nullptr, rows, f->H, f->eps, 1.f / L.in_scale, f->x.codes, f->x.sf, true, f->stream));
    Fp4GemmCall gu;
    gu.X = &f->x, gu.W = &L.gate, gu.W2 = &L.up;
    gu.alpha = L.in_scale * L.s_gate, gu.alpha2 = L.in_scale * L.s_up;
    gu.q_out = f->mid.codes, gu.sf_out = f->mid.sf, gu.sf_out_tiled = true, gu.gscale_out = 1.f / L.mid_scale;
    gu.err_flag = f->err, gu.ctas = f->ctas;
    LB_TRY(fp4_gemm_launch(gu, f->stream));
    Fp4GemmCall dn;
    dn.X = &f->mid, dn.W = &L.down;
    dn.alpha = L.mid_scale * L.s_down;
    dn.y = f->h, dn.ldy = f->H, dn.accumulate = true;
    dn.err_flag = f->err, dn.ctas = f->ctas;
    LB_TRY(fp4_gemm_launch(dn, f->stream));
  }
  return LING_B200_OK;
}

}  // namespace

extern "C" {

int ling_b200_quantize_nvfp4_host(int device, const uint16_t* w_bf16, int N, int K, uint8_t* values, uint8_t* scales, float* scale2) {
  if (!w_bf16 || !values || !scales || !scale2 || N < 1 || !multiple(K, 16)) {
    set_error("quantize_nvfp4: K must be a positive multiple of 16");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  auto* w = reinterpret_cast<__nv_bfloat16*>(sc.put(w_bf16, size_t(N) * K));
  uint8_t* q = sc.get<uint8_t>(size_t(N) * (K / 2));
  uint8_t* sf = sc.get<uint8_t>(size_t(N) * (K / 16));
  float* s2 = sc.get<float>(1);
  unsigned* amax = sc.get<unsigned>(1);
  LB_PTR(w && q && sf && s2 && amax);
  LB_TRY(fp4_quant_weight_launch(w, N, K, q, sf, false, s2, amax, 0));
  LB_CUDA(cudaMemcpy(values, q, size_t(N) * (K / 2), cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(scales, sf, size_t(N) * (K / 16), cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(scale2, s2, 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

int ling_b200_quant_act_nvfp4_host(int device, const float* x, const float* up, int M, int K, float input_scale, uint8_t* q, uint8_t* sf) {
  if (!x || !q || !sf || M < 1 || !multiple(K, 16) || !(input_scale > 0.f)) {
    set_error("quant_act_nvfp4: K must be a positive multiple of 16 and input_scale positive");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  float* dx = sc.put(x, size_t(M) * K);
  float* du = up ? sc.put(up, size_t(M) * K) : nullptr;
  uint8_t* dq = sc.get<uint8_t>(size_t(M) * (K / 2));
  uint8_t* ds = sc.get<uint8_t>(size_t(M) * (K / 16));
  LB_PTR(dx && dq && ds && (!up || du));
  LB_TRY(fp4_quant_act_launch(dx, du, M, K, 1.f / input_scale, dq, ds, false, 0));
  LB_CUDA(cudaMemcpy(q, dq, size_t(M) * (K / 2), cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(sf, ds, size_t(M) * (K / 16), cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

int ling_b200_rmsnorm_quant_nvfp4_host(int device, const float* x, const uint16_t* w_bf16, float* out, int M, int H, float eps,
                                       float input_scale, uint8_t* q, uint8_t* sf) {
  if (!x || !w_bf16 || !q || !sf || M < 1 || !multiple(H, 16) || !(input_scale > 0.f)) {
    set_error("rmsnorm_quant: H must be a positive multiple of 16 and input_scale positive");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  float* dx = sc.put(x, size_t(M) * H);
  auto* dw = reinterpret_cast<__nv_bfloat16*>(sc.put(w_bf16, size_t(H)));
  float* dout = out ? sc.get<float>(size_t(M) * H) : nullptr;
  uint8_t* dq = sc.get<uint8_t>(size_t(M) * (H / 2));
  uint8_t* ds = sc.get<uint8_t>(size_t(M) * (H / 16));
  LB_PTR(dx && dw && dq && ds && (!out || dout));
  LB_TRY(fp4_rmsnorm_quant_launch(dx, dw, dout, M, H, eps, 1.f / input_scale, dq, ds, false, 0));
  if (out) LB_CUDA(cudaMemcpy(out, dout, size_t(M) * H * 4, cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(q, dq, size_t(M) * (H / 2), cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(sf, ds, size_t(M) * (H / 16), cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

int ling_b200_prefill_gemm_nvfp4_host(int device, const uint8_t* xq, const uint8_t* xs, int M, const uint8_t* wq, const uint8_t* ws,
                                      float alpha, float* y, int ldy, int N, int K, int accumulate) {
  if (!xq || !xs || !wq || !ws || !y || M < 0 || !multiple(N, 128) || !multiple(K, 128) || ldy < N || ldy % 4) {
    set_error("prefill_gemm_nvfp4: N % 128 and K % 128 must be 0, ldy >= N and a multiple of 4");
    return LING_B200_ERR_ARG;
  }
  if (M == 0) return LING_B200_OK;
  LB_TRY(check_device(device));
  Scratch sc;
  Fp4Operand X, W;
  LB_TRY(upload_operand(sc, X, xq, xs, M, K));
  LB_TRY(upload_operand(sc, W, wq, ws, N, K));
  float* dy = sc.put(y, size_t(M) * ldy);
  int* err = sc.get<int>(1);
  LB_PTR(dy && err);
  Fp4GemmCall c;
  c.X = &X, c.W = &W, c.alpha = alpha, c.y = dy, c.ldy = ldy, c.accumulate = accumulate != 0, c.err_flag = err;
  LB_TRY(fp4_gemm_launch(c, 0));
  LB_CUDA(cudaDeviceSynchronize());
  LB_TRY(read_flag(err, "prefill_gemm_nvfp4"));
  LB_CUDA(cudaMemcpy(y, dy, size_t(M) * ldy * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

int ling_b200_prefill_swiglu_nvfp4_host(int device, const uint8_t* xq, const uint8_t* xs, int M, const uint8_t* gate_q,
                                        const uint8_t* gate_s, float alpha_gate, const uint8_t* up_q, const uint8_t* up_s, float alpha_up,
                                        int N, int K, float out_input_scale, uint8_t* q_out, uint8_t* sf_out) {
  if (!xq || !xs || !gate_q || !gate_s || !up_q || !up_s || !q_out || !sf_out || M < 0 || !multiple(N, 128) || !multiple(K, 128) ||
      !(out_input_scale > 0.f)) {
    set_error("prefill_swiglu_nvfp4: N % 128 and K % 128 must be 0 and out_input_scale positive");
    return LING_B200_ERR_ARG;
  }
  if (M == 0) return LING_B200_OK;
  LB_TRY(check_device(device));
  Scratch sc;
  Fp4Operand X, G, U;
  LB_TRY(upload_operand(sc, X, xq, xs, M, K));
  LB_TRY(upload_operand(sc, G, gate_q, gate_s, N, K));
  LB_TRY(upload_operand(sc, U, up_q, up_s, N, K));
  uint8_t* dq = sc.get<uint8_t>(size_t(M) * (N / 2));
  uint8_t* ds = sc.get<uint8_t>(size_t(M) * (N / 16));
  int* err = sc.get<int>(1);
  LB_PTR(dq && ds && err);
  Fp4GemmCall c;
  c.X = &X, c.W = &G, c.W2 = &U, c.alpha = alpha_gate, c.alpha2 = alpha_up;
  c.q_out = dq, c.sf_out = ds, c.sf_out_tiled = false, c.gscale_out = 1.f / out_input_scale, c.err_flag = err;
  LB_TRY(fp4_gemm_launch(c, 0));
  LB_CUDA(cudaDeviceSynchronize());
  LB_TRY(read_flag(err, "prefill_swiglu_nvfp4"));
  LB_CUDA(cudaMemcpy(q_out, dq, size_t(M) * (N / 2), cudaMemcpyDeviceToHost));
  LB_CUDA(cudaMemcpy(sf_out, ds, size_t(M) * (N / 16), cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

int ling_b200_nvfp4_pair_mode(int mode) { return fp4_set_pair_mode(mode != 0 ? 1 : 0); }

int ling_b200_nvfp4_gemm_bench(int device, int M, int N, int K, int fused, int iters, float* ms_per_launch, double* cycle_shares) {
  if (!ms_per_launch || M < 1 || !multiple(N, 128) || !multiple(K, 128) || iters < 1) {
    set_error("nvfp4_gemm_bench: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  Scratch sc;
  Fp4Operand X, W, W2, Out;
  auto make = [&](Fp4Operand& o, int rows, int Kk, int seed) -> int {
    o.rows = rows, o.K = Kk;
    o.codes = sc.get<uint8_t>(size_t(rows) * (Kk / 2));
    o.sf = sc.get<uint8_t>(fp4_sf_bytes(rows, Kk));
    LB_PTR(o.codes && o.sf);
    // codes: every nibble pattern; scales: E4M3 codes 0x30..0x3f (0.5 .. 1.9)
    std::vector<uint8_t> hq(size_t(rows) * (Kk / 2)), hs(fp4_sf_bytes(rows, Kk));
    uint64_t s = 0x9E3779B97F4A7C15ull * uint64_t(seed + 1);
    for (auto& b : hq) b = uint8_t((s = s * 6364136223846793005ull + 1442695040888963407ull) >> 56);
    for (auto& b : hs) b = uint8_t(0x30 + (((s = s * 6364136223846793005ull + 1442695040888963407ull) >> 60) & 15));
    LB_CUDA(cudaMemcpy(o.codes, hq.data(), hq.size(), cudaMemcpyHostToDevice));
    LB_CUDA(cudaMemcpy(o.sf, hs.data(), hs.size(), cudaMemcpyHostToDevice));
    return make_fp4_map(o);
  };
  LB_TRY(make(X, M, K, 1));
  LB_TRY(make(W, N, K, 2));
  if (fused) LB_TRY(make(W2, N, K, 3));
  float* y = fused ? nullptr : sc.get<float>(size_t(M) * N);
  if (fused) LB_TRY(make(Out, M, N, 4));
  int* err = sc.get<int>(1);
  LB_PTR(err && (fused || y));
  Fp4GemmCall c;
  c.X = &X, c.W = &W, c.W2 = fused ? &W2 : nullptr, c.alpha = 1e-3f, c.alpha2 = 1e-3f;
  c.y = y, c.ldy = N, c.q_out = Out.codes, c.sf_out = Out.sf, c.err_flag = err;
  cudaEvent_t a, b;
  LB_CUDA(cudaEventCreate(&a));
  LB_CUDA(cudaEventCreate(&b));
  for (int i = 0; i < 3; ++i) LB_TRY(fp4_gemm_launch(c, 0));
  LB_CUDA(cudaEventRecord(a, 0));
  for (int i = 0; i < iters; ++i) LB_TRY(fp4_gemm_launch(c, 0));
  LB_CUDA(cudaEventRecord(b, 0));
  LB_CUDA(cudaEventSynchronize(b));
  float t = 0.f;
  LB_CUDA(cudaEventElapsedTime(&t, a, b));
  cudaEventDestroy(a), cudaEventDestroy(b);
  LB_TRY(read_flag(err, "nvfp4_gemm_bench"));
  *ms_per_launch = t / iters;
  if (cycle_shares) {  // one more launch with the kernel's own cycle counters on
    unsigned long long* st = sc.get<unsigned long long>(4);
    LB_PTR(st);
    c.stats = st;
    LB_TRY(fp4_gemm_launch(c, 0));
    unsigned long long h[4];
    LB_CUDA(cudaMemcpy(h, st, sizeof h, cudaMemcpyDeviceToHost));
    for (int i = 0; i < 3; ++i) cycle_shares[i] = h[3] ? double(h[i]) / double(h[3]) : 0.0;
  }
  return LING_B200_OK;
}

// The NVFP4 tensor pipe's dense rate (fp4_tensor_peak_kernel): one CTA per SM, `iters` MMA groups each, timed with CUDA
// events after a warm-up launch; TFLOP/s = 2 * 128 * 256 * 256 * iters * SMs / time.
int ling_b200_fp4_tensor_peak(int device, int iters, int mode, float* tflops, float* ms) {
  if (!tflops || iters < 1 || iters > (1 << 22) || mode < 0 || mode > 4) {
    set_error("fp4_tensor_peak: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  Scratch sc;
  int* err = sc.get<int>(1);
  LB_PTR(err);
  cudaEvent_t a, b;
  LB_CUDA(cudaEventCreate(&a));
  LB_CUDA(cudaEventCreate(&b));
  LB_TRY(fp4_tensor_peak_launch(sms, iters, mode, err, 0));
  LB_CUDA(cudaEventRecord(a, 0));
  LB_TRY(fp4_tensor_peak_launch(sms, iters, mode, err, 0));
  LB_CUDA(cudaEventRecord(b, 0));
  LB_CUDA(cudaEventSynchronize(b));
  float t = 0.f;
  LB_CUDA(cudaEventElapsedTime(&t, a, b));
  cudaEventDestroy(a), cudaEventDestroy(b);
  LB_TRY(read_flag(err, "fp4_tensor_peak"));
  *tflops = float(2.0 * 128 * 256 * 256 * double(iters) * sms / (double(t) * 1e-3) / 1e12);
  if (ms) *ms = t;
  return LING_B200_OK;
}

int ling_b200_nvfp4_ffn_create(int device, int layers, int hidden, int intermediate, int max_rows, uint64_t seed,
                               ling_b200_nvfp4_ffn** out) {
  if (!out || layers < 1 || !multiple(hidden, 256) || !multiple(intermediate, 128) || max_rows < 1) {
    set_error("nvfp4_ffn_create: hidden % 256 and intermediate % 128 must be 0");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  std::unique_ptr<ling_b200_nvfp4_ffn> f(new ling_b200_nvfp4_ffn);
  f->device = device, f->layers = layers, f->H = hidden, f->I = intermediate, f->max_rows = max_rows;
  LB_CUDA(cudaStreamCreateWithFlags(&f->stream, cudaStreamNonBlocking));
  LB_CUDA(cudaEventCreate(&f->ev0));
  LB_CUDA(cudaEventCreate(&f->ev1));
  f->h = f->mem.get<float>(size_t(max_rows) * hidden);
  f->err = f->mem.get<int>(1);
  LB_PTR(f->h && f->err);
  LB_TRY(alloc_operand(f->mem, f->x, max_rows, hidden));
  LB_TRY(alloc_operand(f->mem, f->mid, max_rows, intermediate));
  LB_CUDA(cudaMallocHost(&f->pin_in, size_t(max_rows) * hidden * 4));
  LB_CUDA(cudaMallocHost(&f->pin_out, size_t(max_rows) * hidden * 4));
  Scratch tmp;
  auto* wtmp = tmp.get<__nv_bfloat16>(size_t(intermediate) * hidden, false);
  unsigned* amax = tmp.get<unsigned>(1);
  float* s2 = tmp.get<float>(1);
  LB_PTR(wtmp && amax && s2);
  f->L.resize(layers);
  for (int l = 0; l < layers; ++l) {
    auto& L = f->L[l];
    L.norm = f->mem.get<__nv_bfloat16>(hidden);
    LB_PTR(L.norm);
    LB_TRY(fill_bf16_launch(nullptr, stream_key(seed, weight_stream(l, LING_B200_T_POST_NORM)), 0.02f, 0.f, 1, L.norm, hidden, f->stream));
    LB_TRY(synth_matrix(f.get(), L.gate, intermediate, hidden, stream_key(seed, weight_stream(l, LING_B200_T_GATE)), wtmp, amax, s2, &L.s_gate));
    LB_TRY(synth_matrix(f.get(), L.up, intermediate, hidden, stream_key(seed, weight_stream(l, LING_B200_T_UP)), wtmp, amax, s2, &L.s_up));
    LB_TRY(synth_matrix(f.get(), L.down, hidden, intermediate, stream_key(seed, weight_stream(l, LING_B200_T_DOWN)), wtmp, amax, s2, &L.s_down));
    // Static activation scales as a calibration would leave them: a block's scale E4M3(amax / 6 / input_scale) saturates
    // at 448, so input_scale = A / (6 * 448) represents magnitudes up to A: 16 for the normed residual (unit variance), 64
    // for the gated product.
    L.in_scale = 16.f / (6.f * 448.f);
    L.mid_scale = 64.f / (6.f * 448.f);
  }
  LB_CUDA(cudaStreamSynchronize(f->stream));
  *out = f.release();
  return LING_B200_OK;
}

void ling_b200_nvfp4_ffn_destroy(ling_b200_nvfp4_ffn* f) { delete f; }

// The DeltaNet layers' mixers in front of their feed-forward blocks: every layer except each `full_every`-th (the full-attention
// layers, whose mixer on the prefill path is not built) gets synthetic mixer weights and a zero state; the activation buffers are shared.
int ling_b200_nvfp4_ffn_add_mixers(ling_b200_nvfp4_ffn* f, int k_heads, int v_heads, int full_every, uint64_t seed) {
  if (!f || !gdn_shape_ok(f->H, k_heads, v_heads) || full_every < 0 || !f->mixers.empty()) {
    set_error("nvfp4_ffn_add_mixers: bad argument, or mixers already added");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(f->device));
  LB_TRY(gdn_chunk_init());
  LB_TRY(gdn_buffers_create(f->mem, f->H, k_heads, v_heads, f->max_rows, f->mix));
  Scratch tmp;
  auto* wtmp = tmp.get<__nv_bfloat16>(size_t(std::max(f->mix.C, f->H)) * std::max(f->H, f->mix.Vs), false);
  unsigned* amax = tmp.get<unsigned>(1);
  float* s2 = tmp.get<float>(1);
  LB_PTR(wtmp && amax && s2);
  f->mixers.resize(size_t(f->layers));
  for (int l = 0; l < f->layers; ++l)
    if (full_every == 0 || l % full_every != full_every - 1) LB_TRY(gdn_weights_create(f->mem, f->stream, f->mix, l, seed, wtmp, amax, s2, f->mixers[size_t(l)]));
  LB_CUDA(cudaStreamSynchronize(f->stream));
  return LING_B200_OK;
}

// The full-attention layers' mixers (every `full_every`-th layer of the stack = the same layer of the verify context, which
// must have as many layers): the chunk's rows are positions pos0.. of session `slot`, whose pages the caller has mapped.
int ling_b200_nvfp4_ffn_attach_context(ling_b200_nvfp4_ffn* f, ling_b200_ctx* ctx, int slot, int pos0, int full_every) {
  if (!f || slot < 0 || pos0 < 0 || full_every < 1) {
    set_error("nvfp4_ffn_attach_context: bad argument");
    return LING_B200_ERR_ARG;
  }
  f->attn_ctx = ctx, f->attn_slot = slot, f->attn_pos0 = pos0, f->attn_every = full_every;
  return LING_B200_OK;
}

int ling_b200_nvfp4_ffn_set_residual(ling_b200_nvfp4_ffn* f, const float* h, int rows) {
  if (!f || !h || rows < 1 || rows > f->max_rows) {
    set_error("nvfp4_ffn_set_residual: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(f->device));
  LB_CUDA(cudaMemcpyAsync(f->h, h, size_t(rows) * f->H * 4, cudaMemcpyHostToDevice, f->stream));
  LB_CUDA(cudaStreamSynchronize(f->stream));
  return LING_B200_OK;
}

int ling_b200_nvfp4_ffn_launch(ling_b200_nvfp4_ffn* f, int rows, int repeats) {
  if (!f || rows < 1 || rows > f->max_rows || repeats < 1) {
    set_error("nvfp4_ffn_launch: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(f->device));
  LB_CUDA(cudaEventRecord(f->ev0, f->stream));
  for (int i = 0; i < repeats; ++i) LB_TRY(ffn_run(f, rows));
  LB_CUDA(cudaEventRecord(f->ev1, f->stream));
  return LING_B200_OK;
}

int ling_b200_nvfp4_ffn_set_ctas(ling_b200_nvfp4_ffn* f, int ctas) {
  if (!f || ctas < 0) return LING_B200_ERR_ARG;
  f->ctas = ctas;
  return LING_B200_OK;
}

int ling_b200_nvfp4_ffn_wait(ling_b200_nvfp4_ffn* f, float* device_ms) {
  if (!f) return LING_B200_ERR_ARG;
  LB_CUDA(cudaSetDevice(f->device));
  LB_CUDA(cudaEventSynchronize(f->ev1));
  if (device_ms) LB_CUDA(cudaEventElapsedTime(device_ms, f->ev0, f->ev1));
  return read_flag(f->err, "nvfp4_ffn");
}

int ling_b200_nvfp4_ffn_forward(ling_b200_nvfp4_ffn* f, const float* h_in, int rows, float* h_out) {
  if (!f || !h_in || !h_out || rows < 1 || rows > f->max_rows) {
    set_error("nvfp4_ffn_forward: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(f->device));
  const size_t bytes = size_t(rows) * f->H * 4;
  std::memcpy(f->pin_in, h_in, bytes);
  LB_CUDA(cudaMemcpyAsync(f->h, f->pin_in, bytes, cudaMemcpyHostToDevice, f->stream));
  LB_TRY(ffn_run(f, rows));
  LB_CUDA(cudaMemcpyAsync(f->pin_out, f->h, bytes, cudaMemcpyDeviceToHost, f->stream));
  LB_CUDA(cudaStreamSynchronize(f->stream));
  LB_TRY(read_flag(f->err, "nvfp4_ffn_forward"));
  std::memcpy(h_out, f->pin_out, bytes);
  return LING_B200_OK;
}

int ling_b200_nvfp4_ffn_read_layer(ling_b200_nvfp4_ffn* f, int layer, uint16_t* norm_bf16, uint8_t* gate_q, uint8_t* gate_s,
                                   uint8_t* up_q, uint8_t* up_s, uint8_t* down_q, uint8_t* down_s, float* scales5) {
  if (!f || layer < 0 || layer >= f->layers) {
    set_error("nvfp4_ffn_read_layer: bad layer");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(f->device));
  const auto& L = f->L[layer];
  Scratch sc;
  auto read = [&](const Fp4Operand& o, uint8_t* q, uint8_t* s) -> int {
    if (q) LB_CUDA(cudaMemcpy(q, o.codes, size_t(o.rows) * (o.K / 2), cudaMemcpyDeviceToHost));
    if (s) {
      uint8_t* raw = sc.get<uint8_t>(size_t(o.rows) * (o.K / 16));
      LB_PTR(raw);
      LB_TRY(fp4_sf_untile_launch(o.sf, raw, o.rows, o.K, 0));
      LB_CUDA(cudaMemcpy(s, raw, size_t(o.rows) * (o.K / 16), cudaMemcpyDeviceToHost));
    }
    return LING_B200_OK;
  };
  if (norm_bf16) LB_CUDA(cudaMemcpy(norm_bf16, L.norm, size_t(f->H) * 2, cudaMemcpyDeviceToHost));
  LB_TRY(read(L.gate, gate_q, gate_s));
  LB_TRY(read(L.up, up_q, up_s));
  LB_TRY(read(L.down, down_q, down_s));
  if (scales5) scales5[0] = L.in_scale, scales5[1] = L.mid_scale, scales5[2] = L.s_gate, scales5[3] = L.s_up, scales5[4] = L.s_down;
  return LING_B200_OK;
}

// ------------------------------------------------------------------------------------------------ a DeltaNet layer's mixer, prefill path
// Engine::forward's linear-attention branch for many rows (src/core/engine.cpp, the quantized path: rmsnorm + NVFP4
// projections, gdn_conv_prefill, gdn_gating, gdn_recurrent_prefill, gated_rmsnorm, out projection) with synthetic weights:
// h += out( gated_norm( delta_rule( conv(in_qkv(norm(h))) ), in_z(norm(h)) ) ).
}  // extern "C"

struct ling_b200_prefill_gdn {
  int device = 0;
  GdnBuffers b;
  GdnWeights w;
  float* h = nullptr;
  int* err = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  Scratch mem;
  ~ling_b200_prefill_gdn() {
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (stream) cudaStreamDestroy(stream);
  }
};

namespace {
int gdn_layer_run(ling_b200_prefill_gdn* f, int rows) { return gdn_mixer_run(f->b, f->w, f->h, rows, f->err, 0, f->stream); }
}  // namespace

extern "C" {

int ling_b200_prefill_gdn_create(int device, int hidden, int k_heads, int v_heads, int max_rows, uint64_t seed, ling_b200_prefill_gdn** out) {
  if (!out || !gdn_shape_ok(hidden, k_heads, v_heads) || max_rows < 1) {
    set_error("prefill_gdn_create: hidden, the mixer's channels and its value width must be multiples of 256 (heads of 128)");
    return LING_B200_ERR_ARG;
  }
  LB_TRY(check_device(device));
  LB_TRY(gdn_chunk_init());
  std::unique_ptr<ling_b200_prefill_gdn> f(new ling_b200_prefill_gdn);
  f->device = device;
  LB_CUDA(cudaStreamCreateWithFlags(&f->stream, cudaStreamNonBlocking));
  LB_CUDA(cudaEventCreate(&f->ev0));
  LB_CUDA(cudaEventCreate(&f->ev1));
  f->h = f->mem.get<float>(size_t(max_rows) * hidden), f->err = f->mem.get<int>(1);
  LB_PTR(f->h && f->err);
  LB_TRY(gdn_buffers_create(f->mem, hidden, k_heads, v_heads, max_rows, f->b));
  Scratch tmp;
  auto* wtmp = tmp.get<__nv_bfloat16>(size_t(std::max(f->b.C, hidden)) * std::max(hidden, f->b.Vs), false);
  unsigned* amax = tmp.get<unsigned>(1);
  float* s2 = tmp.get<float>(1);
  LB_PTR(wtmp && amax && s2);
  LB_TRY(gdn_weights_create(f->mem, f->stream, f->b, 0, seed, wtmp, amax, s2, f->w));
  LB_CUDA(cudaStreamSynchronize(f->stream));
  *out = f.release();
  return LING_B200_OK;
}

void ling_b200_prefill_gdn_destroy(ling_b200_prefill_gdn* f) { delete f; }

// The session's state [HV][128][128] and conv window [C][3]: set (NULL: zero) or read back.
int ling_b200_prefill_gdn_state(ling_b200_prefill_gdn* f, int write, float* state, float* conv) {
  if (!f) return LING_B200_ERR_ARG;
  LB_CUDA(cudaSetDevice(f->device));
  const size_t sb = size_t(f->b.HV) * 128 * 128 * 4, cb = size_t(f->b.C) * 3 * 4;
  if (write) {
    if (state) LB_CUDA(cudaMemcpyAsync(f->w.state, state, sb, cudaMemcpyHostToDevice, f->stream));
    else LB_CUDA(cudaMemsetAsync(f->w.state, 0, sb, f->stream));
    if (conv) LB_CUDA(cudaMemcpyAsync(f->w.conv, conv, cb, cudaMemcpyHostToDevice, f->stream));
    else LB_CUDA(cudaMemsetAsync(f->w.conv, 0, cb, f->stream));
  } else {
    if (state) LB_CUDA(cudaMemcpyAsync(state, f->w.state, sb, cudaMemcpyDeviceToHost, f->stream));
    if (conv) LB_CUDA(cudaMemcpyAsync(conv, f->w.conv, cb, cudaMemcpyDeviceToHost, f->stream));
  }
  LB_CUDA(cudaStreamSynchronize(f->stream));
  return LING_B200_OK;
}

// h [rows][hidden] in, the layer's mixer applied (h += ...), h out; the state and the window advance.
int ling_b200_prefill_gdn_forward(ling_b200_prefill_gdn* f, const float* h_in, int rows, float* h_out) {
  if (!f || !h_in || !h_out || rows < 1 || rows > f->b.max_rows) {
    set_error("prefill_gdn_forward: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(f->device));
  const size_t bytes = size_t(rows) * f->b.H * 4;
  LB_CUDA(cudaMemcpyAsync(f->h, h_in, bytes, cudaMemcpyHostToDevice, f->stream));
  LB_TRY(gdn_layer_run(f, rows));
  LB_CUDA(cudaMemcpyAsync(h_out, f->h, bytes, cudaMemcpyDeviceToHost, f->stream));
  LB_CUDA(cudaStreamSynchronize(f->stream));
  return read_flag(f->err, "prefill_gdn_forward");
}

// `repeats` passes over the resident residual, timed on the device (ms in all); the state keeps advancing.
int ling_b200_prefill_gdn_bench(ling_b200_prefill_gdn* f, int rows, int repeats, float* ms) {
  if (!f || rows < 1 || rows > f->b.max_rows || repeats < 1 || !ms) {
    set_error("prefill_gdn_bench: bad argument");
    return LING_B200_ERR_ARG;
  }
  LB_CUDA(cudaSetDevice(f->device));
  LB_TRY(gdn_layer_run(f, rows));
  LB_CUDA(cudaEventRecord(f->ev0, f->stream));
  for (int i = 0; i < repeats; ++i) LB_TRY(gdn_layer_run(f, rows));
  LB_CUDA(cudaEventRecord(f->ev1, f->stream));
  LB_CUDA(cudaEventSynchronize(f->ev1));
  LB_CUDA(cudaEventElapsedTime(ms, f->ev0, f->ev1));
  return read_flag(f->err, "prefill_gdn_bench");
}

// What the last forward left between the stages, for parity checks (any pointer may be NULL): xn [rows][hidden], pre [rows][C],
// z [rows][Vs], g / beta [rows][HV], core [rows][Vs].
int ling_b200_prefill_gdn_read_stages(ling_b200_prefill_gdn* f, int rows, float* xn, float* pre, float* z, float* g, float* beta, float* core) {
  if (!f || rows < 1 || rows > f->b.max_rows) return LING_B200_ERR_ARG;
  LB_CUDA(cudaSetDevice(f->device));
  const size_t R = size_t(rows);
  if (xn) LB_CUDA(cudaMemcpy(xn, f->b.xn, R * f->b.H * 4, cudaMemcpyDeviceToHost));
  if (pre) LB_CUDA(cudaMemcpy(pre, f->b.pre, R * f->b.C * 4, cudaMemcpyDeviceToHost));
  if (z) LB_CUDA(cudaMemcpy(z, f->b.z, R * f->b.Vs * 4, cudaMemcpyDeviceToHost));
  if (g) LB_CUDA(cudaMemcpy(g, f->b.g, R * f->b.HV * 4, cudaMemcpyDeviceToHost));
  if (beta) LB_CUDA(cudaMemcpy(beta, f->b.beta, R * f->b.HV * 4, cudaMemcpyDeviceToHost));
  if (core) LB_CUDA(cudaMemcpy(core, f->b.core, R * f->b.Vs * 4, cudaMemcpyDeviceToHost));
  return LING_B200_OK;
}

// The layer's weights as the device holds them: BF16 bit patterns of the small tensors, and the three NVFP4 matrices (codes
// [N][K/2], block scales row-major [N][K/16]) with their tensor scales; scales5 = {in_scale, mid_scale, s_qkv, s_z, s_out}.
int ling_b200_prefill_gdn_read_weights(ling_b200_prefill_gdn* f, uint16_t* norm, uint16_t* convw, uint16_t* wa, uint16_t* wb, uint16_t* A_log,
                                       uint16_t* dt_bias, uint16_t* lin_norm, uint8_t* qkv_q, uint8_t* qkv_s, uint8_t* z_q, uint8_t* z_s,
                                       uint8_t* out_q, uint8_t* out_s, float* scales5) {
  if (!f) return LING_B200_ERR_ARG;
  LB_CUDA(cudaSetDevice(f->device));
  Scratch sc;
  auto small = [&](uint16_t* dst, const __nv_bfloat16* src, size_t n) -> int {
    if (dst) LB_CUDA(cudaMemcpy(dst, src, n * 2, cudaMemcpyDeviceToHost));
    return LING_B200_OK;
  };
  LB_TRY(small(norm, f->w.norm, f->b.H));
  LB_TRY(small(convw, f->w.convw, size_t(f->b.C) * 4));
  LB_TRY(small(wa, f->w.wa, size_t(f->b.HV) * f->b.H));
  LB_TRY(small(wb, f->w.wb, size_t(f->b.HV) * f->b.H));
  LB_TRY(small(A_log, f->w.A_log, f->b.HV));
  LB_TRY(small(dt_bias, f->w.dt_bias, f->b.HV));
  LB_TRY(small(lin_norm, f->w.lin_norm, 128));
  auto read = [&](const Fp4Operand& o, uint8_t* q, uint8_t* s) -> int {
    if (q) LB_CUDA(cudaMemcpy(q, o.codes, size_t(o.rows) * (o.K / 2), cudaMemcpyDeviceToHost));
    if (s) {
      uint8_t* raw = sc.get<uint8_t>(size_t(o.rows) * (o.K / 16));
      LB_PTR(raw);
      LB_TRY(fp4_sf_untile_launch(o.sf, raw, o.rows, o.K, 0));
      LB_CUDA(cudaMemcpy(s, raw, size_t(o.rows) * (o.K / 16), cudaMemcpyDeviceToHost));
    }
    return LING_B200_OK;
  };
  LB_TRY(read(f->w.in_qkv, qkv_q, qkv_s));
  LB_TRY(read(f->w.in_z, z_q, z_s));
  LB_TRY(read(f->w.out, out_q, out_s));
  if (scales5) scales5[0] = f->b.in_scale, scales5[1] = f->b.mid_scale, scales5[2] = f->w.s_qkv, scales5[3] = f->w.s_z, scales5[4] = f->w.s_out;
  return LING_B200_OK;
}

}  // extern "C"
