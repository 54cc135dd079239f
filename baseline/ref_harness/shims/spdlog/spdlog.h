// Stand-in for the spdlog submodule that the original tree expects under src/external/spdlog (absent from its
// repository snapshot): the logging calls compile to nothing.
#pragma once
namespace spdlog {
template <typename... A> inline void info(const char*, const A&...) {}
template <typename... A> inline void warn(const char*, const A&...) {}
template <typename... A> inline void error(const char*, const A&...) {}
template <typename... A> inline void debug(const char*, const A&...) {}
template <typename... A> inline void critical(const char*, const A&...) {}
}  // namespace spdlog
