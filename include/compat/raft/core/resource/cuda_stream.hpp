#pragma once
#include <raft/core/resources.hpp>
