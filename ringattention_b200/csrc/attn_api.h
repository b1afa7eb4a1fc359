// C ABI of the attention-backward launchers, shared by the translation units that call them.
#pragma once

struct RaAttnBwdArgs {
  const void* q; const void* k; const void* v; const void* d_o;
  long long q_sb, q_ss, q_sh;
  long long k_sb, k_ss, k_sh;
  long long v_sb, v_ss, v_sh;
  long long do_sb, do_ss, do_sh;
  const float* lse2; const float* delta; int Sq_pad;
  float* dq_acc;
  void* dk; void* dv; long long dkv_sb, dkv_ss, dkv_sh; int dkv_mode;
  int B, H, Sq, Sk, D;
  float softmax_scale;
  int causal_block_size;
  int q_off0, q_off1, q_half;
  int k_off0, k_off1, k_half;
  const int* seg_q; const int* seg_k; const int* seg_q_mm; const int* seg_k_mm;
  const float* bias; long long bias_sb, bias_sh;
  unsigned long long seed; unsigned int drop_threshold;
  const unsigned int* keep; long long keep_sb, keep_sh, keep_sr;  // boolean mask bitmap by kv row, or null
  const void* copy_src; void* copy_dst; long long copy_bytes; int copy_ctas;
  int* status;
  void* stream;
  // optional, this launch only: device buffer of 4*64*4 int64 on the launch's device that the first compute CTA
  // fills with SM-clock timestamps of its pipeline phases (null = no tracing)
  long long* trace;
};

extern "C" int ra_attn_bwd(const RaAttnBwdArgs* a);
extern "C" int ra_attn_bwd_prep(const void* o, long long o_sb, long long o_ss, long long o_sh,
                                const void* d_o, long long do_sb, long long do_ss, long long do_sh,
                                const float* lse, float* lse2, float* delta, int B, int H, int Sq,
                                int Sq_pad, int D, void* stream);
extern "C" int ra_cast_f32_bf16(const float* src, void* dst, long long rows, int d, long long src_ld,
                                long long dst_ld, void* stream);
