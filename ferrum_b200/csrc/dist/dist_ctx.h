// Shared definitions of the inter-GPU kernels: the per-rank context that every
// kernel receives by value, and the layout of the flag region at the start of
// each rank's symmetric arena.
#pragma once
#include <stdint.h>

#define FB_MAX_RANKS 8
#define FB_FLAG_CHANNELS 8
#define FB_FLAG_BLOCKS 1024
// flags[channel][block][source rank], one 32-bit epoch each
#define FB_FLAG_WORDS (FB_FLAG_CHANNELS * FB_FLAG_BLOCKS * FB_MAX_RANKS)
#define FB_FLAG_BYTES 262144  // flag words (8 x 1024 x 8 x 4 B), so the data region stays 64 KiB aligned

typedef struct {
  int rank;
  int world;
  // Base of every rank's arena as seen from THIS rank (index = rank); entry [rank] is local memory.
  unsigned char* arena[FB_MAX_RANKS];
  // NVSwitch multicast alias of the arenas (NULL when multicast is not set up).
  unsigned char* mc_arena;
  int32_t* status;                // host-mapped status block (may be NULL)
  unsigned long long timeout_ns;  // bound of every wait on a peer flag
} fb_dist_ctx;

enum {
  FB_COLL_BROADCAST = 0,
  FB_COLL_ALL_GATHER = 1,
  FB_COLL_GATHER = 2,
  FB_COLL_SCATTER = 3,
  FB_COLL_REDUCE_SCATTER = 4,
  FB_COLL_REDUCE = 5,
  FB_COLL_ALL_GATHER_INPLACE = 6,  // rank p's chunk already sits at in_off + p * n_bytes on rank p
};
enum { FB_OP_SUM = 0, FB_OP_PROD = 1, FB_OP_MIN = 2, FB_OP_MAX = 3, FB_OP_AVG = 4 };
enum { FB_FUSE_NONE = 0, FB_FUSE_SGD = 1, FB_FUSE_ADAM = 2 };
