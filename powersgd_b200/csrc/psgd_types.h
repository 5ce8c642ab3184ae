// Plain-C descriptors shared between the host planner (Python, numpy structured arrays)
// and the device kernels. All offsets are in floats. Keep in sync with ops/layout.py.
#pragma once
#include <stdint.h>

#define PSGD_MAX_RANK 32   // largest factor rank the kernels are instantiated for
#define PSGD_MAX_HIST 8    // largest num_iters_per_step
#define PSGD_CMAT_STRIDE (PSGD_MAX_RANK * PSGD_MAX_RANK)

// One compressed gradient matrix (row-major n x m, contiguous rows).
typedef struct {
  float* grad;    // gradient + carried residual on entry; local residual on exit
  float* param;   // parameter (fused SGD) or null
  float* mom;     // momentum buffer (fused SGD) or null
  float* out;     // averaged low-rank gradient or null
  int32_t n, m, r;
  int32_t p_off, q_off;          // this matrix's [n,r] / [m,r] block inside P-/Q-shaped buffers
  int32_t grp_p_off, grp_p_len;  // whole shape group's block (rank-1 joint normalisation)
  int32_t grp_q_off, grp_q_len;
  int32_t hyper;                 // row of the hyper-parameter table
  int32_t index;                 // position of this matrix in the descriptor array
  int32_t pad0;
} PsgdMat;  // 80 bytes

// One unit of work of the two product kernels.
typedef struct {
  int32_t mat;
  int32_t row0, rows;
  int32_t col0, cols;
  int32_t split, nsplit;   // this tile's position among the tiles whose partial sums are added
  int32_t ticket;          // index of the arrival counter shared by those tiles
  int32_t slot0;           // first partial-sum slot of that set (slot = slot0 + split)
  int32_t vec;             // floats per global access the matrix allows: 4 (16-byte aligned rows),
                           // 2 (8-byte aligned rows, e.g. a row pitch of 650 floats) or 1
  int32_t pad[2];
} PsgdTile;  // 48 bytes

// SGD hyper-parameters of one parameter group (read on the device every step, so the
// host can change the learning rate without rebuilding anything).
typedef struct {
  float lr, momentum, one_minus_dampening, weight_decay;
  int32_t nesterov, has_momentum;
  float grad_scale;
  int32_t pad;
} PsgdHyper;  // 32 bytes

// One slice of a flat (uncompressed) tensor list.
typedef struct {
  float* grad;
  float* param;
  float* mom;
  float* out;
  int64_t numel;
  int64_t flat_off;  // offset inside the flat communication buffer
  int32_t hyper;
  int32_t op;        // per-item operation of a mixed launch (psgd_flat_launch mode 9): 8 or 5
  int32_t pad[2];
} PsgdFlat;  // 64 bytes
