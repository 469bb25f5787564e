// Host-side interface between the C ABI (qmk_api.cu) and the batched decode kernel (qmk_batch.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/qmk_b200.h"

struct qmk_batch_ctx;

// Checks the descriptor against what the batched kernel supports (QMK_OK or QMK_ERR_UNSUPPORTED_MODEL).
int qmkb_supported(const qmk_model_desc* d);

// Phases of one decode step for this descriptor (5 per layer, MoE 6, plus the LM head).
int qmkb_num_phases(const qmk_model_desc* d);

// Builds the tensor maps of the weight matrices and allocates the scratch on the current device.
int qmkb_create(const qmk_model_desc* d, const qmk_weight_ptrs* w, int n_sm, qmk_batch_ctx** out, char* err, size_t errlen);
void qmkb_destroy(qmk_batch_ctx* c);

struct qmkb_launch_args {
  int pos;                 // position of every row when the state has no position_ids
  int phase_begin, phase_end;
  int wait_first;
  int cooperative;
  long long timeout_cycles;
  unsigned long long* trace;   // optional timeline buffer (qmk_set_trace), or null
};
// One launch of phases [phase_begin, phase_end) (plus the memset of the arrival counters before it).
int qmkb_launch(qmk_batch_ctx* c, const qmk_state_ptrs* st, const qmkb_launch_args* a, cudaStream_t stream, char* err,
                size_t errlen);

// Device status record (8 words) and a full reset of the scratch after a failed launch.
unsigned* qmkb_status_ptr(qmk_batch_ctx* c);
int qmkb_reset(qmk_batch_ctx* c, cudaStream_t stream);
const int* qmkb_expert_count_ptr(const qmk_batch_ctx* c);   // device address of the step's distinct-expert count, or null
// Device addresses of what the last router phase left: the distinct experts in ascending order [E] and the router
// weight of every (slot, row) [E, 64] (0 where the row did not pick the expert); null for a dense model.
const int* qmkb_expert_list_ptr(const qmk_batch_ctx* c);
unsigned long long* qmkb_expert_reads_ptr(const qmk_batch_ctx* c);   // device counter: distinct experts over all router phases
const float* qmkb_expert_weight_ptr(const qmk_batch_ctx* c);
// Expert parallelism: exchange buffer of this rank (allocated on first call; its inter-process handle) and the peers' buffers.
int qmkb_ep_export(qmk_batch_ctx* c, void* ipc_handle_out, char* err, size_t errlen);
int qmkb_ep_connect(qmk_batch_ctx* c, const void* ipc_handles, char* err, size_t errlen);
void qmkb_geometry(const qmk_batch_ctx* c, int* ctas, int* threads, int* smem_bytes);
size_t qmkb_scratch_bytes(const qmk_batch_ctx* c);
