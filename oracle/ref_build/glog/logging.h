// Minimal stand-in for <glog/logging.h>, used only to compile the reference's own
// attention sources (tensor, buffer, allocators and the three CUDA files on the decode
// attention path) into oracle/_ref/ as a parity checker. glog itself is not installed in
// the build image. Only the macros those sources use are provided: CHECK, CHECK_EQ/NE/
// LT/LE/GT/GE, LOG(severity), LOG_IF(severity, cond). A failed CHECK or a FATAL message
// prints the streamed text and aborts, which is glog's behaviour.
//
// TEST INFRASTRUCTURE ONLY: nothing in the product library includes this header.
#ifndef ORACLE_REF_BUILD_GLOG_LOGGING_H
#define ORACLE_REF_BUILD_GLOG_LOGGING_H

// glog.h pulls these in transitively and the reference headers rely on that.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>
#include <iostream>
#include <sstream>

namespace glog_standin {

enum Severity { SEV_INFO = 0, SEV_WARNING = 1, SEV_ERROR = 2, SEV_FATAL = 3 };

class Message {
public:
    Message(const char* file, int line, int severity) : severity_(severity) {
        static const char* tags[] = {"I", "W", "E", "F"};
        text_ << tags[severity] << " " << file << ":" << line << "] ";
    }
    ~Message() {
        if (severity_ >= SEV_ERROR) {
            std::cerr << text_.str() << std::endl;
        }
        if (severity_ == SEV_FATAL) {
            std::abort();
        }
    }
    std::ostream& stream() { return text_; }

private:
    int severity_;
    std::ostringstream text_;
};

// Lets `cond ? (void)0 : Voidify() & stream` type-check, the usual trick for
// conditional logging statements that still accept `<<`.
struct Voidify {
    void operator&(std::ostream&) {}
};

}  // namespace glog_standin

#define GLOG_STANDIN_SEV_INFO ::glog_standin::SEV_INFO
#define GLOG_STANDIN_SEV_WARNING ::glog_standin::SEV_WARNING
#define GLOG_STANDIN_SEV_ERROR ::glog_standin::SEV_ERROR
#define GLOG_STANDIN_SEV_FATAL ::glog_standin::SEV_FATAL

#define LOG(sev) ::glog_standin::Message(__FILE__, __LINE__, GLOG_STANDIN_SEV_##sev).stream()
#define LOG_IF(sev, cond) \
    !(cond) ? (void)0 : ::glog_standin::Voidify() & LOG(sev)

#define CHECK(cond) LOG_IF(FATAL, !(cond)) << "Check failed: " #cond " "
#define GLOG_STANDIN_CHECK_OP(a, b, op) \
    LOG_IF(FATAL, !((a)op(b))) << "Check failed: " #a " " #op " " #b " "
#define CHECK_EQ(a, b) GLOG_STANDIN_CHECK_OP(a, b, ==)
#define CHECK_NE(a, b) GLOG_STANDIN_CHECK_OP(a, b, !=)
#define CHECK_LT(a, b) GLOG_STANDIN_CHECK_OP(a, b, <)
#define CHECK_LE(a, b) GLOG_STANDIN_CHECK_OP(a, b, <=)
#define CHECK_GT(a, b) GLOG_STANDIN_CHECK_OP(a, b, >)
#define CHECK_GE(a, b) GLOG_STANDIN_CHECK_OP(a, b, >=)

#endif  // ORACLE_REF_BUILD_GLOG_LOGGING_H
