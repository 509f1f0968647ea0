// Stand-in for <spdlog/spdlog.h>, used only when the reference's kernel sources
// are compiled in place for the parity harness. The reference logs a profile
// summary through spdlog::info; the harness needs no logging, so these swallow
// their arguments.
#pragma once
namespace spdlog {
template <typename... Args> inline void info(Args&&...) {}
template <typename... Args> inline void warn(Args&&...) {}
template <typename... Args> inline void error(Args&&...) {}
template <typename... Args> inline void debug(Args&&...) {}
}  // namespace spdlog
