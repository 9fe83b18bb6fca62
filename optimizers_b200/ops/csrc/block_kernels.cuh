// Grouped per-block kernels of the optimizer step: one launch covers every block of a
// parameter group through a device block table.
//
//   grad_prologue       one read of the gradient produces everything the step needs from it:
//                       L2-regularised gradient, its tf32 (hi, lo) split in both orientations
//                       (the K-major operands of the factor Gram GEMMs), the filtered-gradient
//                       EMA and its bias-corrected, split form (operand of the preconditioner
//                       GEMMs), the diagonal second moment of the grafting method, the squared
//                       norm of the grafting direction, and a non-finite status flag.
//   direction_epilogue  grafting rescale, weight decay, classic momentum, multiplication by -lr,
//                       primal averaging and the parameter update (or the cast into the
//                       all-gather send buffer) in one pass.
//
// They replace the chains of torch._foreach_* launches of the reference
// (distributed_shampoo/distributed_shampoo.py:1110-1139, :1170-1199, :1232-1293, :1358-1381,
// :1484; preconditioner/adagrad_preconditioner_list.py:122-162;
// distributor/shampoo_distributor.py:361-365).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace ob200 {

// One 2-D block (m x n).  1-D blocks are presented as 1 x n; a contiguous order-3 block (a, b, c)
// as (a*b) x c, plus an auxiliary descriptor a x (b*c) for the operand layouts of the other modes.
struct BlockDesc {
  float* param;        // view into the parameter; element (i, j) at param[i * param_pitch + j]
  long long param_pitch;
  long long grad_offset;  // element offset of the block inside its parameter's gradient
  int grad_slot;          // index into the per-step gradient pointer array
  int m, n;
  int n_pad, m_pad;       // row pitches of the row-major / transposed split arrays
  float* m1;              // filtered gradient EMA [m, n] (null if beta1 == 0)
  float* v;               // diagonal second moment [m, n] (null unless AdaGrad-family grafting)
  float* mom;             // classic momentum buffer [m, n] (null if unused)
  float* z;               // primal-averaging weight buffer [m, n] (null if unused)
  float* g_hi;            // [m, n_pad]  (null if dim 0 has no factor)
  float* g_lo;
  float* gt_hi;           // [n, m_pad]  (null if dim 1 has no factor)
  float* gt_lo;
  float* f_hi;            // filtered gradient, bias corrected, [m, n_pad]
  float* f_lo;
  float* p;               // search direction [m, n] (output of the preconditioner GEMMs)
  float* norms;           // [2]: squared norm of the grafting direction, of the Shampoo direction
  void* send;             // all-gather send slot in the communication dtype (null: update params)
  long long slot_offset;  // byte offset of the block's slot inside the gather buffer (peer push)
  float* ev;              // eigenvalue-corrected second moment [m, n] (null unless SOAP)
  int aux;                // 1: a second 2-D view of an order-3 block that only needs the operand
                          // splits of its gradient (g_*, gt_*); it carries no state (m1, v, f_* and
                          // norms are null) and the epilogue kernels skip it
                          // 2: a block none of whose dims is preconditioned: the prologue writes the
                          // filtered gradient to p and its squared norm to norms[1] itself
  int pad_;
};

struct TileRef {
  int block;
  int ti;  // 32-row tile index
  int tj;  // 128-column tile index
  int pad_;
};

enum GraftKind : int { kGraftNone = 0, kGraftSGD = 1, kGraftAdaGrad = 2 };

struct PrologueArgs {
  const BlockDesc* blocks;
  const TileRef* tiles;
  int num_tiles;
  const float* const* grad_ptrs;  // [slot * max(num_grad_peers, 1) + r]: gradient base pointers
  int num_grad_peers;             // 0: local gradient; G > 0: the gradient is the scaled sum of G
                                  // ranks' gradients, loaded from peer memory over NVLink in rank
                                  // order (reduce-scatter fused into the owner's prologue)
  float grad_scale;               // 1 / G for a mean
  float l2_weight_decay;          // 0 unless WeightDecayType.L2
  float beta1, beta3;
  float bias_correction1;         // 1 - beta3 * beta1^(t-1), or 1
  int graft_kind;
  float graft_beta2, graft_weight, graft_bias_correction2, graft_epsilon;
  int write_split;                // 0: store raw fp32 into the *_hi arrays and skip *_lo (tf32 mode)
  int* status;                    // bit 1 set when a gradient holds NaN/Inf
};

struct EpilogueArgs {
  const BlockDesc* blocks;
  const TileRef* tiles;
  int num_tiles;
  const float* lr;                // device scalar
  int graft_only;                 // direction = grafting direction (before start_preconditioning_step)
  int graft_kind;
  float graft_bias_correction2, graft_epsilon;
  float wd_alpha;                 // decoupled-style weight decay coefficient (0: none)
  int primal_averaging;
  const float* mu_y;              // train interpolation coefficient (device scalar)
  const float* mu_x;              // eval interpolation coefficient (device scalar)
  int classic_momentum;
  float momentum, dampening;
  int nesterov;
  int send_dtype;                 // 0 fp32, 1 bf16, 2 fp16 (only with BlockDesc::send)
  int split_input;                // f given as (hi, lo) pair (1) or raw in f_hi (0)
  int num_push_peers;             // G > 0: store the direction into the gather buffer of all G ranks
                                  // (all-gather fused into the epilogue); 0: BlockDesc::send or params
  unsigned long long peer_base[8];  // gather-buffer base address on each rank (this rank included)
  int send_params;                // 1: what is sent is the updated parameter W + update (communicate_params)
};

// eig_scale: S = P / ((ev / bc2)^(1/root) + eps) on the projected filtered gradient held in
// BlockDesc::p, written as the (hi, lo) operand pair into f_hi / f_lo for the unprojection GEMMs
// (reference: shampoo_preconditioner_list.py:1920-1942).
void launch_eig_scale(const BlockDesc* blocks, const TileRef* tiles, int num_tiles, float bias_correction2,
                      float inv_root, float epsilon, int write_split, cudaStream_t stream);

// mode_switch: W <- W + c (Z - W) for every block, the train()/eval() switch of the primal
// averaging schemes; with BlockDesc::send the delta goes to the gather buffer instead
// (reference: distributed_shampoo.py:1749-1757, :1783-1794).
void launch_mode_switch(const BlockDesc* blocks, const TileRef* tiles, int num_tiles, float coeff, int send_dtype,
                        cudaStream_t stream);

constexpr int kErrGemmTimeout = 1;  // grouped GEMM: a bounded pipeline wait expired (kErrPipelineTimeout)
constexpr int kErrPeerTimeout = 4;  // a bounded wait on a peer's flag expired

// Cross-rank barrier over peer memory: writes `seq` into slot `my_rank` of every peer's flag
// array, then waits (bounded) until every slot of the local flag array has reached `seq`.
void launch_peer_barrier(int* local_flags, const unsigned long long* peer_flag_bases, int my_rank, int world,
                         int seq, int* status, cudaStream_t stream);

void launch_grad_prologue(const PrologueArgs& args, cudaStream_t stream);
void launch_direction_epilogue(const EpilogueArgs& args, cudaStream_t stream);

// gathered_apply: after the all-gather every rank adds each block's direction, read from its
// slot of the receive buffer in the communication dtype (BlockDesc::send points at the slot),
// to the parameter block.  One grouped launch replaces the reference's _foreach_add_ over views
// of the gather buffer (distributed_shampoo/distributor/shampoo_ddp_distributor.py:330-360).
// With `lr` non-null the slots hold unscaled directions P and BlockDesc::norms points at the
// block's grafting scale s: W <- W - lr (s P + wd_alpha W); this finishes, on every rank, the
// update whose directions the preconditioner GEMM pushed from its epilogue.
// `copy_params`: the slots hold updated parameters (communicate_params): W <- slot.
// `status` (may be null): the group's device status word; when a timeout bit is set in it the
// kernel leaves the parameters untouched.
void launch_gathered_apply(const BlockDesc* blocks, const TileRef* tiles, int num_tiles, int dtype, const float* lr,
                           float wd_alpha, bool copy_params, const int* status, cudaStream_t stream);

}  // namespace ob200
