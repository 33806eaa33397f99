// Which problems the TMA + tcgen05 kernels take, and the switch over the three ops.
#include "common.h"

namespace limn_b200 {

int tcgen05_fwd(const Problem& p);
int tcgen05_bwd_q(const Problem& p);
int tcgen05_bwd_kv(const Problem& p);

bool tcgen05_serves(Op op, const Problem& p) {
  if (p.dtype != LIMN_B200_BF16 && p.dtype != LIMN_B200_F16) return false;
  // built for head dims 64 and 128; narrower heads (hd for Q and K, hd_v for V) run in the next of the two with their
  // missing columns read as zeros
  if (p.hd < 8 || p.hd > 128 || p.hd % 8 != 0 || p.hd_v < 8 || p.hd_v > 128 || p.hd_v % 8 != 0) return false;
  if (!(p.scale > 0.0)) return false;          // the softmax folds the scale into exp2 and takes row maxima before scaling
  if (p.bh > 0x7fffffffLL) return false;       // problem index is a 32-bit TMA coordinate
  return true;
}

int tcgen05_launch(Op op, const Problem& p) {
  switch (op) {
    case Op::Fwd: return tcgen05_fwd(p);
    case Op::BwdQ: return tcgen05_bwd_q(p);
    case Op::BwdKV: return tcgen05_bwd_kv(p);
  }
  return fail(LIMN_B200_UNSUPPORTED, "sdpa: no tcgen05 kernel for this op");
}

}  // namespace limn_b200
