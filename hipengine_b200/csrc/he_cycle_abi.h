// Control block of the native speculative-cycle / decode-step launcher.
//
// The host runtime hands one of these to he_cycle_launch() together with an instantiated CUDA graph.  The
// launcher checks the block (magic, version, size, stage mask, bounds), launches the graph on the given stream,
// optionally waits for it, and fills the bounded result block.  It performs no device math of its own.
// Role of the reference's native cycle ABI (hipengine/speculative/native_cycle_abi.h: a versioned, fixed-size
// control block with a stage mask PROPOSE / VERIFY / ACCEPT / COMMIT / UPDATE_CURSORS and chain / tree mode).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HE_CYCLE_MAGIC 0x48454359u /* 'HECY' */
#define HE_CYCLE_VERSION 1u
#define HE_CYCLE_MAX_REQUESTS 64u
#define HE_CYCLE_MAX_DEPTH 16u

enum HeCycleStage {
  HE_STAGE_PROPOSE = 1u << 0,
  HE_STAGE_VERIFY = 1u << 1,
  HE_STAGE_ACCEPT = 1u << 2,
  HE_STAGE_COMMIT = 1u << 3,
  HE_STAGE_UPDATE_CURSORS = 1u << 4,
  HE_STAGE_DECODE_STEP = 1u << 5, /* plain autoregressive step captured as one graph */
};

enum HeCycleMode { HE_MODE_CHAIN = 0, HE_MODE_TREE = 1 };

typedef struct HeCycleControlV1 {
  uint32_t magic;        /* HE_CYCLE_MAGIC */
  uint32_t version;      /* HE_CYCLE_VERSION */
  uint32_t struct_bytes; /* sizeof(HeCycleControlV1): catches drift between the two sides of the ABI */
  uint32_t stage_mask;   /* which stages the captured graph contains */
  uint32_t mode;         /* HeCycleMode; only HE_MODE_CHAIN is accepted */
  uint32_t n_requests;   /* 1 .. HE_CYCLE_MAX_REQUESTS */
  uint32_t depth;        /* draft tokens per request, 0 .. HE_CYCLE_MAX_DEPTH (0 for a decode step) */
  uint32_t wait;         /* 1: synchronise the stream before returning */
  uint64_t status_word;  /* device pointer (int*) that kernels write a non-zero code to, or 0 */
  uint64_t n_accept;     /* device pointer (int32[n_requests]) read back when wait != 0, or 0 */
  uint64_t reserved[4];
} HeCycleControlV1;

typedef struct HeCycleResultV1 {
  int32_t rc;             /* 0, a negative HeStatus code, or a positive cudaError_t */
  int32_t device_status;  /* value of *status_word after the cycle (wait != 0 only) */
  int32_t n_accept[HE_CYCLE_MAX_REQUESTS];
  uint64_t launches;      /* graphs launched through this entry point since load */
} HeCycleResultV1;

int he_cycle_control_size(void);
int he_cycle_result_size(void);
int he_cycle_validate(const HeCycleControlV1* c);

#ifdef __cplusplus
}
#endif
