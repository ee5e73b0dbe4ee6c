// Stand-in for ppl.common's log.h: LOG(LEVEL) << ... writes one line to stderr.
// See retcode.h in this directory.
#ifndef PPLB200_COMPAT_PPL_COMMON_LOG_H
#define PPLB200_COMPAT_PPL_COMMON_LOG_H

#include <iostream>
#include <sstream>

namespace ppl { namespace common {

enum { LOG_LEVEL_DEBUG = 0, LOG_LEVEL_INFO, LOG_LEVEL_WARNING, LOG_LEVEL_ERROR, LOG_LEVEL_FATAL };

class LogLine final {
public:
    LogLine(int level, const char* file, int line) : level_(level) {
        static const char* tags[] = {"DEBUG", "INFO", "WARNING", "ERROR", "FATAL"};
        os_ << "[" << tags[level] << "][" << file << ":" << line << "] ";
    }
    ~LogLine() {
        if (level_ >= LOG_LEVEL_WARNING) std::cerr << os_.str() << std::endl;
    }
    template <typename T>
    LogLine& operator<<(const T& v) { os_ << v; return *this; }

private:
    int level_;
    std::ostringstream os_;
};

}}

#define LOG(LEVEL) ::ppl::common::LogLine(::ppl::common::LOG_LEVEL_##LEVEL, __FILE__, __LINE__)

#endif
