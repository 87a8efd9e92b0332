// TEST INFRASTRUCTURE.  C entry points around the reference's own knowledge-graph container
// (smore/cpp_sampler/src/lib/knowledge_graph.cpp, compiled where it lies together with utils.cpp; see
// oracle/build.py), so that files written by smore_b200/kg_format.py can be checked against the
// reference: it builds the alias tables of a weight vector (AliasMethod), builds a graph from triplets and dumps it (KG::load_from_numpy, KG::dump), loads a
// file (KG::load) and answers edge / degree queries from it.  Built without NDEBUG: the reference
// does its file I/O inside assert().
#include <cstdint>
#include <string>

#include "alias_method.h"
#include "knowledge_graph.h"

template <typename D>
static int build_and_dump(const int64_t* triplets, size_t n, uint64_t num_ent, uint64_t num_rel, int has_reverse,
                          const char* path) {
  KG<D> kg((D)num_ent, (D)num_rel);
  kg.load_from_numpy(const_cast<int64_t*>(triplets), n, has_reverse != 0);
  kg.dump(path);
  return 0;
}

template <typename D>
static int load_and_query(const char* path, const int64_t* queries, size_t n_queries, int64_t* answers, uint64_t* stats) {
  KG<D> kg;
  kg.load(path);
  stats[0] = kg.num_ent;
  stats[1] = kg.num_rel;
  stats[2] = kg.num_edges;
  stats[3] = kg.max_degree();
  // every query is (src, rel, dst): answers = {forward edge?, backward edge?, out degree of src, in degree of src}
  for (size_t i = 0; i < n_queries; ++i) {
    const D s = (D)queries[3 * i], r = (D)queries[3 * i + 1], d = (D)queries[3 * i + 2];
    answers[4 * i] = kg.has_forward_edge(s, r, d);
    answers[4 * i + 1] = kg.has_backward_edge(s, r, d);
    answers[4 * i + 2] = kg.out_degree(s);
    answers[4 * i + 3] = kg.in_degree(s);
  }
  return 0;
}

// The reference's alias tables for `weights` (AliasMethod::setup -> build_table, alias_method.cpp:55-99).
struct AliasProbe : AliasMethod {
  using AliasMethod::choice_large;
  using AliasMethod::choice_small;
  using AliasMethod::prob_small;
};

extern "C" {
int ref_alias_build(const double* weights, size_t n, double* prob_small, int64_t* choice_small, int64_t* choice_large) {
  std::vector<double> w(weights, weights + n);
  AliasProbe am;
  am.setup(w);
  for (size_t i = 0; i < n; ++i) {
    prob_small[i] = am.prob_small[i];
    choice_small[i] = (int64_t)am.choice_small[i];
    choice_large[i] = (int64_t)am.choice_large[i];
  }
  return 0;
}

int ref_kg_build_and_dump(const int64_t* triplets, size_t n, uint64_t num_ent, uint64_t num_rel, int has_reverse,
                          int use64, const char* path) {
  return use64 ? build_and_dump<uint64_t>(triplets, n, num_ent, num_rel, has_reverse, path)
               : build_and_dump<unsigned>(triplets, n, num_ent, num_rel, has_reverse, path);
}
int ref_kg_load_and_query(const char* path, int use64, const int64_t* queries, size_t n_queries, int64_t* answers,
                          uint64_t* stats) {
  return use64 ? load_and_query<uint64_t>(path, queries, n_queries, answers, stats)
               : load_and_query<unsigned>(path, queries, n_queries, answers, stats);
}
}
