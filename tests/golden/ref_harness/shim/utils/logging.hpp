// Stand-in for the reference's utils/logging.hpp (which needs the plog submodule): no-op log streams.
#pragma once
#include <cstdio>
#include <ostream>
#include <string>
namespace zedinfer::utils {
enum { FILE_ONLY = 0, CONSOLE_ONLY = 1, BOTH = 2 };
struct NullLog {
    template <typename T> NullLog& operator<<(const T&) { return *this; }
    NullLog& operator<<(std::ostream& (*)(std::ostream&)) { return *this; }
    template <typename... A> void printf(const char*, A...) {}
};
}  // namespace zedinfer::utils
#define LOGE ::zedinfer::utils::NullLog()
#define LOGW ::zedinfer::utils::NullLog()
#define LOGI ::zedinfer::utils::NullLog()
#define LOGD ::zedinfer::utils::NullLog()
#define LOGV ::zedinfer::utils::NullLog()
#define LOGF ::zedinfer::utils::NullLog()
#define LOGE_(x) ::zedinfer::utils::NullLog()
#define LOGW_(x) ::zedinfer::utils::NullLog()
#define LOGI_(x) ::zedinfer::utils::NullLog()
#define LOGD_(x) ::zedinfer::utils::NullLog()
#define LOGV_(x) ::zedinfer::utils::NullLog()
#define PLOG_ERROR ::zedinfer::utils::NullLog()
#define PLOG_WARNING ::zedinfer::utils::NullLog()
#define PLOG_INFO ::zedinfer::utils::NullLog()
#define PLOG_DEBUG ::zedinfer::utils::NullLog()
#define LOG_ERROR_(x) ::zedinfer::utils::NullLog()
#define LOG_WARNING_(x) ::zedinfer::utils::NullLog()
#define LOG_INFO_(x) ::zedinfer::utils::NullLog()
#define LOG_DEBUG_(x) ::zedinfer::utils::NullLog()
#define LOG_VERBOSE_(x) ::zedinfer::utils::NullLog()
#define LOG_FATAL_(x) ::zedinfer::utils::NullLog()
#define LOG_ERROR ::zedinfer::utils::NullLog()
#define LOG_WARNING ::zedinfer::utils::NullLog()
#define LOG_INFO ::zedinfer::utils::NullLog()
#define LOG_DEBUG ::zedinfer::utils::NullLog()
