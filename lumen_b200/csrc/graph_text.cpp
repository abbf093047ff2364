#include "graph_text.h"

#include <sstream>

namespace lb {

std::string TensorType::str() const {
    std::string s = std::string(dtype_name(dtype)) + "[";
    for (size_t d = 0; d < shape.size(); d++) s += (d ? "," : "") + std::to_string(shape[d]);
    return s + "]";
}

const std::string& Node::attr(const std::string& key) const {
    auto it = attrs.find(key);
    if (it == attrs.end()) fail(LB_ERR_INVALID, op + ": missing attribute " + key);
    return it->second;
}
std::vector<int64_t> Node::ints(const std::string& key) const { return parse_int_list(attr(key)); }
int64_t Node::integer(const std::string& key) const { return std::stoll(attr(key)); }

std::vector<int64_t> parse_int_list(const std::string& text) {
    std::vector<int64_t> out;
    if (text.empty() || text == "-") return out;
    size_t at = 0;
    while (at <= text.size()) {
        size_t comma = text.find(',', at);
        if (comma == std::string::npos) comma = text.size();
        out.push_back(std::stoll(text.substr(at, comma - at)));
        at = comma + 1;
    }
    return out;
}

Module parse_module(const std::string& text) {
    Module m;
    std::shared_ptr<Graph> g;
    std::istringstream lines(text);
    std::string line;
    int line_no = 0;
    auto define = [&](int id, const std::string& dtype, const std::string& shape, int node) {
        if (!g) fail(LB_ERR_INVALID, format("graph text line %d: value outside a graph", line_no));
        if (id < 0 || id > (1 << 24)) fail(LB_ERR_INVALID, format("graph text line %d: bad value id", line_no));
        if ((int)g->types.size() <= id) {
            g->types.resize(id + 1);
            g->producer.resize(id + 1, -1);
        }
        g->types[id].dtype = dtype_from_name(dtype);
        g->types[id].shape = parse_int_list(shape);
        g->producer[id] = node;
    };
    while (std::getline(lines, line)) {
        line_no++;
        std::istringstream ts(line);
        std::vector<std::string> tok;
        for (std::string t; ts >> t;) tok.push_back(t);
        if (tok.empty()) continue;
        const std::string& kind = tok[0];
        if (kind == "option" && tok.size() == 2) {
            m.options.insert(tok[1]);
        } else if (kind == "graph") {
            g = std::make_shared<Graph>();
        } else if (kind == "in" && tok.size() == 4) {
            define(std::stoi(tok[1]), tok[2], tok[3], -1);
            g->inputs.push_back(std::stoi(tok[1]));
        } else if (kind == "node" && tok.size() >= 6) {
            Node n;
            n.output = std::stoi(tok[1]);
            n.op = tok[2];
            for (auto v : parse_int_list(tok[5])) n.inputs.push_back((int)v);
            for (size_t k = 6; k < tok.size(); k++) {
                size_t eq = tok[k].find('=');
                if (eq == std::string::npos) fail(LB_ERR_INVALID, format("graph text line %d: bad attribute", line_no));
                n.attrs[tok[k].substr(0, eq)] = tok[k].substr(eq + 1);
            }
            define(n.output, tok[3], tok[4], (int)g->nodes.size());
            for (int v : n.inputs)
                if (v < 0 || v >= (int)g->types.size())
                    fail(LB_ERR_INVALID, format("graph text line %d: %%%d used before it is defined", line_no, v));
            g->nodes.push_back(std::move(n));
        } else if (kind == "out" && tok.size() == 2) {
            for (auto v : parse_int_list(tok[1])) g->outputs.push_back((int)v);
        } else if (kind == "end") {
            if (!g) fail(LB_ERR_INVALID, "graph text: 'end' without 'graph'");
            m.graphs.push_back(g);
            g.reset();
        } else {
            fail(LB_ERR_INVALID, format("graph text line %d: cannot parse '%s'", line_no, line.c_str()));
        }
    }
    if (m.graphs.empty()) fail(LB_ERR_INVALID, "graph text: no graph");
    return m;
}

}  // namespace lb
