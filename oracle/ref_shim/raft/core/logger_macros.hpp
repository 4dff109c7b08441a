// Stand-in for the cmake-generated raft/core/logger_macros.hpp (oracle/_ref build only).
#pragma once
#define RAFT_LOG_ACTIVE_LEVEL 6
#define RAFT_LOG_TRACE(...) (void)0
#define RAFT_LOG_DEBUG(...) (void)0
#define RAFT_LOG_INFO(...) (void)0
#define RAFT_LOG_WARN(...) (void)0
#define RAFT_LOG_ERROR(...) (void)0
#define RAFT_LOG_CRITICAL(...) (void)0
