// Stand-in for legate's CPU collective header: declarations only, one rank never calls them.
#pragma once
#include <cstddef>
namespace legate::comm::coll {
enum class CollDataType { CollFloat, CollDouble };
struct Coll_Comm;
using CollComm = Coll_Comm*;
inline int collAlltoall(const void*, void*, std::size_t, CollDataType, CollComm) { return 0; }
inline int collAllgather(const void*, void*, std::size_t, CollDataType, CollComm) { return 0; }
}  // namespace legate::comm::coll
