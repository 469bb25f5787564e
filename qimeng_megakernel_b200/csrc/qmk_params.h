// Kernel parameter block of the decode megakernel (plain data, passed by value as a
// __grid_constant__).  Plays the role of the reference's LlamaGlobals POD
// (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_kernel/globals.cuh:1-277)
// without the CuTe views: raw pointers, strides in elements.
#pragma once
#include <stdint.h>

namespace qmk {

// Words of the device status record (mirrors qmk_status in the C ABI).
enum StatusWord : int { kStCode = 0, kStSm = 1, kStWarp = 2, kStPhase = 3, kStSeen = 4, kStExpected = 5, kStDetail = 6 };
// 1: a producer's tagged words never arrived; 2: a weight copy never completed; 3: another warp of the CTA never staged its part;
// 4: (batched kernel) an active row's position lies outside the KV cache or the RoPE table: the row was treated as inactive
enum StatusCode : int { kOkCode = 0, kErrCounterWait = 1, kErrCopyWait = 2, kErrStageWait = 3, kErrRowPosition = 4 };

struct Params {
  // ---- weights (bf16 as raw 16-bit words) ----
  const uint16_t* attn_norm;     // [L, H]
  const uint16_t* qkv;           // [L, QKV_ROWS, H]
  const uint16_t* o_proj;        // [L, H, QDIM]
  const uint16_t* mlp_norm;      // [L, H]
  const uint16_t* up;            // [L, I, H]
  const uint16_t* gate;          // [L, I, H]
  const uint16_t* down;          // [L, H, I]
  const uint16_t* lm_norm;       // [H]
  const uint16_t* lm_head;       // [V, H]
  const uint16_t* embed;         // [V, H]
  const float* rope_cos;         // [rope_rows, HD]
  const float* rope_sin;
  // ---- request state ----
  uint16_t* hidden;              // [H]
  uint16_t* q_post_rope;         // [QDIM]
  uint16_t* k_cache;             // [L, B, S, NKV, HD]
  uint16_t* v_cache;
  uint16_t* attn_out;            // [QDIM]
  uint16_t* silu_out;            // [I]
  uint16_t* logits;              // [V]
  long long* next_token;         // optional
  const long long* token_in;     // optional
  long long* out_tokens;         // optional, written at [pos+1]
  long long out_tokens_len;
  long long kv_layer_stride;     // elements between layers (= B*S*NKV*HD)
  long long kv_seq_stride;       // elements between positions (= NKV*HD)
  // ---- library-owned scratch ----
  unsigned long long* part_rec;  // [NH, kMaxSplits, HD + 2] split-KV partial records, words {fp32 bits, tag}
  // tagged activation words {low 16: bf16 value, high 16: tag of (step, phase)}: the cross-SM hand-off
  uint32_t* t_hid_o;             // [H]   residual stream after the O-projection
  uint32_t* t_hid_d;             // [H]   residual stream after the down-projection
  uint32_t* t_q;                 // [QDIM + 2*NKV*HD]  q_post_rope, then this step's K row and V row
  uint32_t* t_attn;              // [QDIM] attention output
  uint32_t* t_silu;              // [I]   SwiGLU output
  unsigned* tickets;             // lm-head arrival ticket at [64]
  unsigned long long* argmax_key;  // packed (ordered logit bits << 32) | ~index
  unsigned* status;              // [8] status words
  unsigned long long* trace;     // optional [CTAs, num_phases, 8] globaltimer stamps (ns); null = off
  // ---- scalars ----
  int num_layers;
  int vocab;
  int pos;                       // position of the token being fed (to the launch's first step)
  int phase_begin, phase_end;    // phases executed by this launch (by every step of it)
  int stream_end;                // where the weight stream of the launch ends: phase_end + (n_steps - 1) * phases per step
  int sync;                      // 1: phases hand off through tagged words; 0: single phase, stream-ordered
  int wait_first;                // 1: also wait for the dependency of phase_begin (debug / failure test)
  unsigned launch_seq;           // number of this launch's first step (per handle): makes every step's tags distinct
  int n_steps;                   // decode steps run by this launch (> 1: whole steps only; step i is position pos + i, fed
                                 // the arg-max of step i - 1 through tok_word)
  unsigned long long* tok_word;  // {token id, tag = number of the step that produced it + 1}: the token hand-off between
                                 // the steps of one launch
  float eps;
  float scale_log2e;             // attn_scale * log2(e)
  long long timeout_cycles;      // bounded-wait budget
};

}  // namespace qmk
