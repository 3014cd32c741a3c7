// Stand-in for the reference's common/logging.h when its mjdgemm sources are compiled on their own
// (test infrastructure).  Only the four macros those sources use exist here: messages go to stderr,
// ABORT ends the process the way the reference's does.
#pragma once
#include <cstdio>
#include <cstdlib>

#define LOG(level, ...) do { std::fprintf(stderr, "[mjdgemm " #level "] %s\n", #__VA_ARGS__); } while(0)
#define LOG_ONCE(level, ...) do { } while(0)
#define ABORT(...) do { std::fprintf(stderr, "[mjdgemm abort] %s\n", #__VA_ARGS__); std::abort(); } while(0)
#define ABORT_IF(cond, ...) do { if(cond) { ABORT(__VA_ARGS__); } } while(0)
