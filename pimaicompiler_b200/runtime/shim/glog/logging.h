// Build shim: the reference's IR and compiler include <glog/logging.h>, which this toolchain does not have.  libtorch
// ships the same macro family (LOG, CHECK, DLOG, ...) in c10/util/Logging.h; the comparison checks glog adds on top are
// defined here.  Found first on the include path when the reference's sources are compiled where they lie.
#pragma once
#include <c10/util/Logging.h>

#include <cstring>
#include <iostream>

#ifndef DLOG
#define DLOG(severity) LOG(severity)
#endif
#ifndef CHECK_LT
#define CHECK_LT(a, b) CHECK((a) < (b))
#define CHECK_LE(a, b) CHECK((a) <= (b))
#define CHECK_GT(a, b) CHECK((a) > (b))
#define CHECK_GE(a, b) CHECK((a) >= (b))
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define CHECK_NE(a, b) CHECK((a) != (b))
#endif
