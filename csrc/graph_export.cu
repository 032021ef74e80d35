// Walk a captured CUDA graph and write it as Graphviz DOT text: one node per graph node
// (kernel nodes carry the kernel's name, launch shape and dynamic shared memory), one edge
// per dependency; programmatic-dependent-launch edges are dashed.  A summary per kernel
// name (launch count) is written as a comment header, which doubles as a launch inventory
// of a decode step.
//
// Plays the role of the reference's graph dump (pegainfer-core/src/cuda_graph/dump.rs:76-569:
// node/edge walk, kernel names, DOT + optional PNG).
#include <stdio.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "api.h"
#include "common.cuh"

namespace {

const char* node_type_name(cudaGraphNodeType t) {
  switch (t) {
    case cudaGraphNodeTypeKernel: return "kernel";
    case cudaGraphNodeTypeMemcpy: return "memcpy";
    case cudaGraphNodeTypeMemset: return "memset";
    case cudaGraphNodeTypeHost: return "host";
    case cudaGraphNodeTypeGraph: return "child graph";
    case cudaGraphNodeTypeEmpty: return "empty";
    case cudaGraphNodeTypeWaitEvent: return "wait event";
    case cudaGraphNodeTypeEventRecord: return "event record";
    case cudaGraphNodeTypeMemAlloc: return "mem alloc";
    case cudaGraphNodeTypeMemFree: return "mem free";
    default: return "node";
  }
}

// "ns::kernel<T>(args...)" -> "kernel<T>": drop the parameter list and leading namespaces
std::string short_name(const char* full) {
  std::string s(full ? full : "?");
  int depth = 0;
  size_t cut = s.size();
  for (size_t i = 0; i < s.size(); ++i) {
    if (s[i] == '<') ++depth;
    else if (s[i] == '>') --depth;
    else if (s[i] == '(' && depth == 0) {
      cut = i;
      break;
    }
  }
  s = s.substr(0, cut);
  depth = 0;
  size_t start = 0;
  for (size_t i = 0; i + 1 < s.size(); ++i) {
    if (s[i] == '<') ++depth;
    else if (s[i] == '>') --depth;
    else if (depth == 0 && s[i] == ':' && s[i + 1] == ':') start = i + 2;
  }
  const size_t sp = s.rfind(' ', start);  // "void name" -> "name"
  (void)sp;
  s = s.substr(start);
  const size_t blank = s.find(' ');
  if (blank != std::string::npos && s.compare(0, 5, "void ") == 0) s = s.substr(5);
  return s;
}

std::string escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') o.push_back('\\');
    o.push_back(c);
  }
  return o;
}

}  // namespace

// counts: [0] nodes, [1] edges, [2] kernel nodes, [3] programmatic edges (may be nullptr).
extern "C" int pg_graph_export_dot(void* graph_ptr, const char* path, const char* title, long long* counts) {
  cudaGraph_t graph = (cudaGraph_t)graph_ptr;
  PG_REQUIRE(graph != nullptr && path != nullptr, "graph export: null graph or path");
  size_t n = 0;
  PG_CUDA(cudaGraphGetNodes(graph, nullptr, &n));
  std::vector<cudaGraphNode_t> nodes(n);
  if (n) PG_CUDA(cudaGraphGetNodes(graph, nodes.data(), &n));
  std::map<cudaGraphNode_t, size_t> index;
  for (size_t i = 0; i < n; ++i) index[nodes[i]] = i;
  size_t ne = 0;
  PG_CUDA(cudaGraphGetEdges_v2(graph, nullptr, nullptr, nullptr, &ne));
  std::vector<cudaGraphNode_t> from(ne), to(ne);
  std::vector<cudaGraphEdgeData> edata(ne);
  if (ne) PG_CUDA(cudaGraphGetEdges_v2(graph, from.data(), to.data(), edata.data(), &ne));

  std::vector<std::string> labels(n);
  std::map<std::string, int> per_kernel;
  long long kernels = 0;
  for (size_t i = 0; i < n; ++i) {
    cudaGraphNodeType t;
    PG_CUDA(cudaGraphNodeGetType(nodes[i], &t));
    char buf[512];
    if (t == cudaGraphNodeTypeKernel) {
      cudaKernelNodeParams kp;
      memset(&kp, 0, sizeof(kp));
      std::string name = "kernel";
      if (cudaGraphKernelNodeGetParams(nodes[i], &kp) == cudaSuccess) {
        const char* full = nullptr;
        if (kp.func != nullptr && cudaFuncGetName(&full, kp.func) == cudaSuccess && full != nullptr) name = short_name(full);
        else (void)cudaGetLastError();
        snprintf(buf, sizeof(buf), "%zu: %s\\ngrid %ux%ux%u block %u smem %u", i, escape(name).c_str(), kp.gridDim.x, kp.gridDim.y, kp.gridDim.z, kp.blockDim.x,
                 kp.sharedMemBytes);
      } else {
        (void)cudaGetLastError();
        snprintf(buf, sizeof(buf), "%zu: kernel", i);
      }
      per_kernel[name] += 1;
      ++kernels;
    } else {
      snprintf(buf, sizeof(buf), "%zu: %s", i, node_type_name(t));
    }
    labels[i] = buf;
  }
  FILE* f = fopen(path, "w");
  PG_REQUIRE(f != nullptr, "graph export: cannot open %s", path);
  long long prog = 0;
  fprintf(f, "// %s: %zu nodes (%lld kernels), %zu edges\n", title ? title : "cuda graph", n, kernels, ne);
  std::vector<std::pair<int, std::string>> order;
  for (auto& kv : per_kernel) order.push_back({kv.second, kv.first});
  std::sort(order.begin(), order.end(), [](const std::pair<int, std::string>& a, const std::pair<int, std::string>& b) { return a.first > b.first || (a.first == b.first && a.second < b.second); });
  for (auto& o : order) fprintf(f, "//   %5d x %s\n", o.first, o.second.c_str());
  fprintf(f, "digraph \"%s\" {\n  rankdir=TB;\n  node [shape=box, fontname=\"monospace\", fontsize=9];\n", escape(title ? title : "cuda graph").c_str());
  for (size_t i = 0; i < n; ++i) fprintf(f, "  n%zu [label=\"%s\"];\n", i, labels[i].c_str());
  for (size_t e = 0; e < ne; ++e) {
    const bool programmatic = edata[e].type == cudaGraphDependencyTypeProgrammatic;
    prog += programmatic ? 1 : 0;
    fprintf(f, "  n%zu -> n%zu%s;\n", index[from[e]], index[to[e]], programmatic ? " [style=dashed]" : "");
  }
  fprintf(f, "}\n");
  fclose(f);
  if (counts) {
    counts[0] = (long long)n;
    counts[1] = (long long)ne;
    counts[2] = kernels;
    counts[3] = prog;
  }
  return PG_OK;
}
