// Symmetric-heap context handed to the P2P collective kernels (mirrored by ctypes in parallel/symm.py).
#pragma once
#include <stdint.h>

#define SYMM_MAX_RANKS 8
#define SYMM_MAX_SLOTS 64
// flag pad size in 32-bit words: ready/done (16 per slot) + epoch (1 per slot) + two block counters (1 each per slot)
#define SYMM_FLAG_WORDS (SYMM_MAX_SLOTS * 19)

struct SymmCtx {
  unsigned char* heap[SYMM_MAX_RANKS];   // base of every rank's heap slab, as mapped on THIS GPU
  uint32_t* flags[SYMM_MAX_RANKS];       // base of every rank's flag pad, as mapped on THIS GPU
  int rank, world;
  unsigned long long wait_ns;            // limit of every wait on a peer flag
};
