// raft::Apply (reference: core/types.hpp:16).
#pragma once
namespace raft {
enum class Apply { ALONG_ROWS, ALONG_COLUMNS };
}  // namespace raft
