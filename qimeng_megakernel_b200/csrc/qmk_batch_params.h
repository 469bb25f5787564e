// Parameter block of the batched decode megakernel (qmk_batch_kernel.cuh): runtime shapes, B sequences
// per step.  Plays the role of the reference's multi-batch globals POD
// (qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/multi_batch/decode_kernel/mk.h:9-42: the
// single-batch tensors with a leading [B] dimension plus position_ids / active_mask) and of the Qwen3
// additions q_norm_weights / k_norm_weights (qimeng_megakernel/models/LLM/qwen/qwen3__0_6b/A100/
// single_batch/decode_kernel/mk.h:7,18-19), as raw pointers.
#pragma once
#include <stdint.h>

namespace qmkb {

constexpr int kMaxBatch = 64;          // sequences per step (N of the tensor-core tile)
constexpr int kTileRows = 128;         // weight rows per tile (M of the tensor-core tile)
constexpr int kBlockK = 64;            // bf16 elements per k-block: 128 bytes, one swizzle row
constexpr int kMaxSplits = 64;         // split-KV partials per (sequence, kv head)

// Phase kinds inside a layer; phase index = layer * ppl + position in the layer (ppl = 5, MoE: 6), the LM head is last.
enum Kind : int { kQkv = 0, kAttn = 1, kOproj = 2, kUpGate = 3, kDown = 4, kLmHead = 5,
                  // MoE layers (six phases: QKV, attention, O-proj, router, expert up/gate, expert down)
                  kRouter = 6, kEUpGate = 7, kEDown = 8 };

struct BParams {
  // ---- weights that are read with plain loads (the matrices come through tensor maps) ----
  const uint16_t* attn_norm;     // [L, H]
  const uint16_t* mlp_norm;      // [L, H]
  const uint16_t* lm_norm;       // [H]
  const uint16_t* q_norm;        // [L, HD] or null (per-head RMSNorm on Q before RoPE)
  const uint16_t* k_norm;        // [L, HD] or null
  const uint16_t* embed;         // [V, H] or null
  const float* rope_cos;         // [rope_rows, HD] interleaved
  const float* rope_sin;
  // ---- request state, bf16 ----
  uint16_t* hidden;              // [B, H]
  uint16_t* q_post_rope;         // [B, QDIM]
  uint16_t* k_cache;             // [L, Bc, S, NKV, HD]
  uint16_t* v_cache;
  uint16_t* attn_out;            // [B, QDIM]
  uint16_t* silu_out;            // [B, I]
  uint16_t* logits;              // [B, V]
  long long* next_token;         // [B] or null
  const long long* token_in;     // [B] or null
  long long* out_tokens;         // [B, out_tokens_len] or null; written at [b, pos_b + 1]
  long long out_tokens_len;
  const int* position_ids;       // [B] or null (then every row is at `pos`)
  const unsigned char* active_mask;   // [B] or null (then every row is active)
  const int* kv_slots;           // [B] or null: the sequence of the KV cache row b reads and appends to (null: sequence b)
  int kv_batch;                  // sequences in the KV cache
  long long kv_layer_stride, kv_batch_stride, kv_seq_stride;   // elements
  // ---- library-owned scratch ----
  long long* ws;                 // [CTAs, Bpad, 128] fixed-point accumulators of split tiles (zero between uses)
  unsigned* tile_tickets;        // [row tiles]   arrivals of a tile's partial segments
  float* ss;                     // [H/128, kMaxBatch]  sums of squares of the residual stream, per row tile
  float* attn_part;              // [items, G, HD + 2]  split-KV partials (acc, max, sum)
  unsigned* attn_tickets;        // [B * NKV]
  unsigned long long* argmax_key;   // [B]  (ordered logit bits << 32) | ~row
  unsigned* phase_done;          // [1 + phases]  CTAs that finished the prologue / each phase (zeroed per launch)
  unsigned* status;              // [8]
  // MoE (null / 0 otherwise): what the router phase leaves for the two expert phases of its layer
  int* moe_ne;                   // [1]  distinct experts selected by the active rows of this step
  int* moe_elist;                // [E]  their indices, ascending
  unsigned long long* moe_ne_sum; // [1]  distinct experts summed over every router phase since the last reset
  float* moe_w;                  // [E, kMaxBatch]  router weight of (slot, row), 0 where the row did not select it
  // activation operands kept as images of a ring slot's activation half: [k-block][Bpad rows][128 bytes, swizzled]
  unsigned char* ximg;           // H / 64 k-blocks: the normalised residual stream (router phase, or a pre-pass)
  unsigned char* aimg;           // QDIM / 64 k-blocks: the attention output (written by the attention phase)
  unsigned char* simg;           // I / 64 k-blocks: SiLU(gate) * up (written by the up/gate epilogue)
  unsigned* img_done;            // [phases]  k-blocks of ximg built by the pre-pass of a phase (zeroed per launch)
  int pre_bpad;                  // normalised layer phases use the pre-pass from this padded batch on
  int pre_lm_units;              // the LM head uses it when a CTA has at least this many units
  int dense_img;                 // O-proj / down-proj read aimg / simg (when their producer ran in the launch)
  unsigned char* eimg;           // selected-expert slot * (Ie / 64) + k-block: SiLU(gate) * up * router weight
  unsigned long long* trace;     // optional [CTAs, phases, 16] timeline words; null = off
  // ---- expert parallelism (ep_world > 1): every rank holds E / ep_world experts, attention and router are replicated;
  // after its local expert down-projection a rank stores each finished [128 rows, Bpad] fp32 partial tile into its slot
  // of every peer's exchange buffer (plain peer stores over NVLink), publishes a flag, waits (bounded) on its OWN
  // buffer's flags and sums the slots in rank order.  Buffer of a rank: [2 (layer parity), ep_world (source), tiles,
  // 128, Bpad] floats, flags [2, ep_world, tiles] words holding the tag of (launch, layer).
  float* ep_buf[8];              // exchange buffer of every rank as mapped into this process (own included)
  unsigned* ep_flag[8];
  int ep_rank, ep_world;         // expert parallelism: which experts the router lists (1 / 0 when off)
  int x_world, x_rank;           // ranks that exchange partial tiles (expert or tensor parallelism; 1 / 0 when off)
  int x_per_layer;               // exchanges per layer: 1 (expert down-projection) or 2 (O-proj and down-proj: tensor parallelism)
  unsigned long long* ep_key[8]; // tensor parallelism: [source rank, 64] arg-max keys of the ranks' vocabulary slices
  unsigned* ep_kflag[8];         // [source rank] tag (launch) of the keys
  int vocab_offset;              // global row of this rank's first LM-head row (tensor parallelism; else 0)
  int embed_rows;                // rows of the embedding table (the whole vocabulary also when the LM head is a slice)
  // ---- shape ----
  int H, I, NH, NKV, HD, QKV_ROWS, QDIM, num_layers, vocab;
  int E, topk, Ie;               // MoE: experts, experts per token, expert intermediate size (E = 0: dense model)
  int ppl;                       // phases per layer: 5 (dense) or 6 (MoE)
  int B, Bpad;                   // sequences, padded to a multiple of 16
  int pos;                       // position of every row when position_ids is null
  int pos_limit;                 // min(kv_seq_len, rope_rows): an active row at or beyond it is switched off and reported
  int phase_begin, phase_end;
  int stages, stage_bytes, off_stages, exch_stride;   // shared-memory plan for this Bpad (smem_plan)
  int prologue;                  // 0 none; 1 sums of squares of `hidden`; 2 embed token_in, then sums of squares
  unsigned epoch;                // number of this launch (per context): tags of the expert-parallel exchange
  int wait_first;                // failure test: the first phase waits for a dependency nothing publishes
  float eps, qk_eps, scale_log2e;
  long long timeout_cycles;
};

}  // namespace qmkb
