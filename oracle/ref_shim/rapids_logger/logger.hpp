// Stand-in for rapids_logger/logger.hpp (oracle/_ref build only): a logger that drops everything.
#pragma once
#include <memory>
#include <string>
#include <vector>

#define RAPIDS_LOGGER_LOG_LEVEL_TRACE 0
#define RAPIDS_LOGGER_LOG_LEVEL_DEBUG 1
#define RAPIDS_LOGGER_LOG_LEVEL_INFO 2
#define RAPIDS_LOGGER_LOG_LEVEL_WARN 3
#define RAPIDS_LOGGER_LOG_LEVEL_ERROR 4
#define RAPIDS_LOGGER_LOG_LEVEL_CRITICAL 5
#define RAPIDS_LOGGER_LOG_LEVEL_OFF 6

namespace rapids_logger {
enum class level_enum : int { trace = 0, debug, info, warn, error, critical, off };
struct sink {
  virtual ~sink() = default;
};
using sink_ptr = std::shared_ptr<sink>;
struct basic_file_sink_mt : sink {
  basic_file_sink_mt(const std::string&, bool) {}
};
struct stderr_sink_mt : sink {};
class logger {
 public:
  logger(std::string, std::vector<sink_ptr>) {}
  void set_pattern(const std::string&) {}
  void set_level(level_enum) {}
  level_enum level() const { return level_enum::off; }
  bool should_log(level_enum) const { return false; }
  void flush() {}
  template <typename... A>
  void log(A&&...)
  {
  }
};
}  // namespace rapids_logger
