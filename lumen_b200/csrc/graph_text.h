// Parser of the graph text format written by lumen_b200/graph.py (Graph.to_text): the form in which fusion bodies
// and whole graphs reach the backend. Mirrors the reference's Graph/Node/TensorType (lumen/graph/mod.rs) only as
// far as the code generators need: typed values, nodes with string attributes, nested fusion bodies.
#pragma once
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "common.h"

namespace lb {

struct TensorType {
    int dtype = LB_F32;
    std::vector<int64_t> shape;
    int64_t numel() const { return lb::numel(shape); }
    int rank() const { return (int)shape.size(); }
    std::string str() const;
};

struct Node {
    std::string op;
    std::vector<int> inputs;
    int output = -1;
    std::map<std::string, std::string> attrs;

    bool has(const std::string& key) const { return attrs.count(key) != 0; }
    const std::string& attr(const std::string& key) const;
    std::vector<int64_t> ints(const std::string& key) const;
    int64_t integer(const std::string& key) const;
    int dtype(const std::string& key) const { return dtype_from_name(attr(key)); }
};

struct Graph {
    std::vector<TensorType> types;  // by value id
    std::vector<int> inputs, outputs;
    std::vector<Node> nodes;
    std::vector<int> producer;  // value id -> node index, -1 for inputs

    const TensorType& type(int v) const { return types.at(v); }
    const Node* node_of(int v) const { return producer.at(v) < 0 ? nullptr : &nodes[producer[v]]; }
};

struct Module {
    std::vector<std::shared_ptr<Graph>> graphs;  // bodies first, the main graph last
    std::set<std::string> options;               // `option <name>` lines (e.g. inplace: an output aliases an input)
    const Graph& main() const { return *graphs.back(); }
};

std::vector<int64_t> parse_int_list(const std::string& text);
Module parse_module(const std::string& text);

}  // namespace lb
