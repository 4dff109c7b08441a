// raft::linalg::NormType (reference: linalg/norm_types.hpp:13-23).
#pragma once
namespace raft {
namespace linalg {
enum NormType : unsigned short { L0PseudoNorm = 0, L1Norm = 1, L2Norm = 2, LinfNorm = 3 };
}  // namespace linalg
}  // namespace raft
