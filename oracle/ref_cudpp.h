// Host stand-in for the slice of the CUDPP library (extra/cudpp in the reference tree, a third-party
// dependency) that the reference's wrapper classes call.  TEST INFRASTRUCTURE.  The prototypes come from
// the reference's own extra/cudpp/include/cudpp.h and cudpp_hash.h; what is restated here is each call's
// observable contract, not CUDPP's algorithms:
//   compact   keeps the flagged elements in their input order and reports how many
//   scan      forward sum, exclusive or inclusive, of ints; reduce = max or sum of ints
//   hash tables (cudpp_hash): a table is built from (key, value) pairs;
//     basic       key -> value;
//     compacting  key -> dense id, ids handed out in ascending key order here (CUDPP's own id order is
//                 an implementation detail the reference never relies on: ids only name chunks);
//     multivalue  the pairs are radix-sorted by key (stable, so equal keys keep their input order), the unique
//                 keys are numbered in ascending order, and a query returns (first position in the sorted
//                 value array, number of values) -- extra/cudpp/src/cudpp_hash/hash_multivalue.cpp:45-110;
//                 cudppMultivalueHashGetIndexCounts, an accessor the reference added to its CUDPP copy,
//                 exposes that (position, count) array in unique-key order.
//   a query for an absent key yields CUDPP_HASH_KEY_NOT_FOUND (0xffffffff), or a zero count.
#pragma once
// (included after the reference's own #include <cudpp.h> / <cudpp_hash.h>; the latter has no include guard)
#include <map>

namespace ref_cudpp {
struct Plan {
  CUDPPConfiguration config;
};
struct Table {
  CUDPPHashTableType type;
  std::map<uint32_t, uint32_t> single;  // basic: value; compacting: id
  std::vector<uint32_t> all_values;     // multivalue: values sorted by key
  std::vector<uint2> index_counts;      // multivalue: per unique key (first position, count)
  std::map<uint32_t, uint32_t> unique;  // multivalue: key -> index into index_counts
};
inline size_t elem_bytes(CUDPPDatatype t) {
  switch (t) {
    case CUDPP_CHAR: case CUDPP_UCHAR: return 1;
    case CUDPP_SHORT: case CUDPP_USHORT: return 2;
    case CUDPP_DOUBLE: case CUDPP_LONGLONG: case CUDPP_ULONGLONG: return 8;
    default: return 4;
  }
}
}  // namespace ref_cudpp

const unsigned int CUDPP_HASH_KEY_NOT_FOUND = 0xffffffffu;

extern "C" {
CUDPPResult cudppCreate(CUDPPHandle *h) { *h = 1; return CUDPP_SUCCESS; }
CUDPPResult cudppDestroy(CUDPPHandle) { return CUDPP_SUCCESS; }
CUDPPResult cudppPlan(const CUDPPHandle, CUDPPHandle *plan, CUDPPConfiguration config, size_t, size_t, size_t) {
  *plan = reinterpret_cast<CUDPPHandle>(new ref_cudpp::Plan{config});
  return CUDPP_SUCCESS;
}
CUDPPResult cudppDestroyPlan(CUDPPHandle plan) {
  delete reinterpret_cast<ref_cudpp::Plan *>(plan);
  return CUDPP_SUCCESS;
}
CUDPPResult cudppCompact(const CUDPPHandle plan, void *d_out, size_t *d_numValid, const void *d_in,
                         const unsigned int *d_isValid, size_t n) {
  const size_t w = ref_cudpp::elem_bytes(reinterpret_cast<ref_cudpp::Plan *>(plan)->config.datatype);
  size_t kept = 0;
  for (size_t i = 0; i < n; ++i)
    if (d_isValid[i]) {
      std::memmove(static_cast<char *>(d_out) + kept * w, static_cast<const char *>(d_in) + i * w, w);
      ++kept;
    }
  *d_numValid = kept;
  return CUDPP_SUCCESS;
}
CUDPPResult cudppScan(const CUDPPHandle plan, void *d_out, const void *d_in, size_t n) {
  const bool inclusive = reinterpret_cast<ref_cudpp::Plan *>(plan)->config.options & CUDPP_OPTION_INCLUSIVE;
  const int *in = static_cast<const int *>(d_in);
  int *out = static_cast<int *>(d_out), acc = 0;
  for (size_t i = 0; i < n; ++i) {
    const int v = in[i];
    out[i] = inclusive ? acc + v : acc;
    acc += v;
  }
  return CUDPP_SUCCESS;
}
CUDPPResult cudppSegmentedScan(const CUDPPHandle plan, void *d_out, const void *d_in, const unsigned int *flags, size_t n) {
  const bool inclusive = reinterpret_cast<ref_cudpp::Plan *>(plan)->config.options & CUDPP_OPTION_INCLUSIVE;
  const int *in = static_cast<const int *>(d_in);
  int *out = static_cast<int *>(d_out), acc = 0;
  for (size_t i = 0; i < n; ++i) {
    if (flags[i]) acc = 0;
    const int v = in[i];
    out[i] = inclusive ? acc + v : acc;
    acc += v;
  }
  return CUDPP_SUCCESS;
}
CUDPPResult cudppReduce(const CUDPPHandle plan, void *d_out, const void *d_in, size_t n) {
  const CUDPPOperator op = reinterpret_cast<ref_cudpp::Plan *>(plan)->config.op;
  const int *in = static_cast<const int *>(d_in);
  int acc = (op == CUDPP_MAX) ? INT32_MIN : 0;
  for (size_t i = 0; i < n; ++i) acc = (op == CUDPP_MAX) ? std::max(acc, in[i]) : acc + in[i];
  *static_cast<int *>(d_out) = acc;
  return CUDPP_SUCCESS;
}

}  // extern "C"  (cudpp_hash.h declares its functions with C++ linkage)

CUDPPResult cudppHashTable(CUDPPHandle, CUDPPHandle *plan, const CUDPPHashTableConfig *config) {
  auto *t = new ref_cudpp::Table();
  t->type = config->type;
  *plan = reinterpret_cast<CUDPPHandle>(t);
  return CUDPP_SUCCESS;
}
CUDPPResult cudppDestroyHashTable(CUDPPHandle, CUDPPHandle plan) {
  delete reinterpret_cast<ref_cudpp::Table *>(plan);
  return CUDPP_SUCCESS;
}
CUDPPResult cudppHashInsert(CUDPPHandle plan, const void *d_keys, const void *d_vals, size_t n) {
  auto *t = reinterpret_cast<ref_cudpp::Table *>(plan);
  const uint32_t *k = static_cast<const uint32_t *>(d_keys), *v = static_cast<const uint32_t *>(d_vals);
  if (t->type == CUDPP_BASIC_HASH_TABLE) {
    for (size_t i = 0; i < n; ++i) t->single[k[i]] = v[i];
  } else if (t->type == CUDPP_COMPACTING_HASH_TABLE) {
    for (size_t i = 0; i < n; ++i) t->single[k[i]] = 0;
    uint32_t id = 0;
    for (auto &kv : t->single) kv.second = id++;
  } else {
    std::vector<size_t> order(n);
    for (size_t i = 0; i < n; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return k[a] < k[b]; });
    t->all_values.resize(n);
    t->index_counts.clear();
    t->unique.clear();
    for (size_t i = 0; i < n; ++i) {
      t->all_values[i] = v[order[i]];
      if (i == 0 || k[order[i]] != k[order[i - 1]]) {
        t->unique[k[order[i]]] = (uint32_t)t->index_counts.size();
        t->index_counts.push_back(uint2{(unsigned)i, 0u});
      }
      t->index_counts.back().y += 1;
    }
  }
  return CUDPP_SUCCESS;
}
CUDPPResult cudppHashRetrieve(CUDPPHandle plan, const void *d_keys, void *d_vals, size_t n) {
  auto *t = reinterpret_cast<ref_cudpp::Table *>(plan);
  const uint32_t *k = static_cast<const uint32_t *>(d_keys);
  if (t->type == CUDPP_MULTIVALUE_HASH_TABLE) {
    uint2 *out = static_cast<uint2 *>(d_vals);
    for (size_t i = 0; i < n; ++i) {
      auto it = t->unique.find(k[i]);
      out[i] = it == t->unique.end() ? uint2{0u, 0u} : t->index_counts[it->second];
    }
  } else {
    uint32_t *out = static_cast<uint32_t *>(d_vals);
    for (size_t i = 0; i < n; ++i) {
      auto it = t->single.find(k[i]);
      out[i] = it == t->single.end() ? CUDPP_HASH_KEY_NOT_FOUND : it->second;
    }
  }
  return CUDPP_SUCCESS;
}
CUDPPResult cudppMultivalueHashGetValuesSize(CUDPPHandle plan, unsigned int *size) {
  *size = (unsigned)reinterpret_cast<ref_cudpp::Table *>(plan)->all_values.size();
  return CUDPP_SUCCESS;
}
CUDPPResult cudppMultivalueHashGetAllValues(CUDPPHandle plan, unsigned int **d_vals) {
  *d_vals = reinterpret_cast<ref_cudpp::Table *>(plan)->all_values.data();
  return CUDPP_SUCCESS;
}
CUDPPResult cudppMultivalueHashGetIndexCounts(CUDPPHandle plan, uint2 **d_index_counts, unsigned *num_unique) {
  auto *t = reinterpret_cast<ref_cudpp::Table *>(plan);
  *d_index_counts = t->index_counts.data();
  *num_unique = (unsigned)t->index_counts.size();
  return CUDPP_SUCCESS;
}
CUDPPResult cudppCompactingHashGetSize(CUDPPHandle plan, unsigned int *size) {
  *size = (unsigned)reinterpret_cast<ref_cudpp::Table *>(plan)->single.size();
  return CUDPP_SUCCESS;
}
