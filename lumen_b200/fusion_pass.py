"""The fusion pass: groups the bare prims of a traced graph into `fusion` nodes, one generated kernel each.

The counterpart of the reference's `fusion` pass for its CUDA device (lumen/graph_compiler/passes/fusion/mod.rs and
README.md; lumen/codegen/fusion/cuda.rs): elementwise chains, reductions with their prologues and epilogues, rows
(several reductions over one row and the elementwise work between and after them: softmax, layer norm, cross
entropy), multi-output fusions, and GEMMs with an elementwise tail (relu, residual add, relu backward) that runs in
the GEMM's epilogue. Like the reference's pass it asks the backend what it can run as one kernel
(`Backend::fusible`, `row_dot`, ... there; `lb_fusion_check` and the compiler's epilogue matcher here) and grows
every group greedily in program order while the answer stays yes.

Graphs whose fusion boundaries were already drawn at trace time (`lumen_b200.nn`) pass through unchanged.
"""

from __future__ import annotations

from lumen_b200 import graph as G

# `gather` (rows of a table picked by an index tensor) is generated inside elementwise kernels like any other load
ELEMENTWISE = set(G.ELEMENTWISE_BINARY) | set(G.FLOAT_UNARY) | set(G.ANY_UNARY) | {"cast", "select", "is_finite", "gather"}
REDUCTIONS = {"reduce_sum", "reduce_max"}
# producers of values out of nothing or of smaller values: cloned into every group that reads them
INLINED = {"full", "iota", "broadcast_in_dim"}
FUSIBLE = ELEMENTWISE | REDUCTIONS | INLINED


def _backend_accepts(body: G.Graph) -> bool:
    """Whether the kernel generator runs `body` as one kernel (no compilation, no GPU needed)."""
    from lumen_b200 import _lib

    return _lib.lib().lb_fusion_check(body.to_text().encode()) == 0


class _Group:
    def __init__(self, gid: int):
        self.gid = gid
        self.members: list[int] = []  # node indices, in program order

    @property
    def last(self) -> int:
        return self.members[-1]


class FusionPass:
    def __init__(self, graph: G.Graph, accepts=_backend_accepts):
        self.g = graph
        self.accepts = accepts
        self.producer = {n.output: i for i, n in enumerate(graph.nodes)}
        self.uses: dict[int, list[int]] = {}
        for i, n in enumerate(graph.nodes):
            for v in n.inputs:
                self.uses.setdefault(v, []).append(i)
        self.outputs = set(graph.outputs)
        self.group_of: dict[int, _Group] = {}  # node index -> group
        self.groups: list[_Group] = []
        self.dot_tail: dict[int, list[int]] = {}  # dot node index -> the elementwise nodes of its epilogue
        # INLINED nodes every reader of which is fusible (directly or through other such nodes): they never become a
        # kernel or a buffer of their own, each group that reads one computes it itself
        self.transparent: set[int] = set()
        # elementwise work on constants alone (`-0.9` of a clamp's bound) is a constant too: cloned, never a group
        constant: set[int] = set()
        for i, n in enumerate(graph.nodes):
            if n.op in ("full", "iota") or (n.op in ELEMENTWISE | {"broadcast_in_dim"} and n.inputs and all(
                    self.producer.get(v) in constant for v in n.inputs)):
                constant.add(i)
        for i in range(len(graph.nodes) - 1, -1, -1):
            n = graph.nodes[i]
            if (n.op in INLINED or i in constant) and n.output not in self.outputs and self.uses.get(n.output) and all(
                    graph.nodes[u].op in ELEMENTWISE | REDUCTIONS or u in self.transparent for u in self.uses[n.output]):
                self.transparent.add(i)

    def readers(self, v: int) -> list[int]:
        """The nodes that read `v`, looking through transparent nodes."""
        out = []
        for u in self.uses.get(v, []):
            out += self.readers(self.g.nodes[u].output) if u in self.transparent else [u]
        return out

    def source_groups(self, v: int) -> list:
        """The groups whose values `v` is computed from, looking through transparent nodes."""
        p = self.producer.get(v)
        if p is None:
            return []
        if p in self.group_of:
            return [self.group_of[p]]
        if p in self.transparent:
            return [grp for x in self.g.nodes[p].inputs for grp in self.source_groups(x)]
        return []

    # ---- bodies ----------------------------------------------------------------------------------------------
    def body_of(self, members: list[int]):
        """The fusion body of `members` (node indices in order) with the INLINED producers they read cloned in.
        Returns (body, outer operands in body-input order, member values that leave the group)."""
        g = self.g
        body = G.Graph()
        inside: dict[int, int] = {}  # outer value -> body value
        operands: list[int] = []

        def value(v: int) -> int:
            if v in inside:
                return inside[v]
            i = self.producer.get(v)
            if i is not None and i in self.transparent:
                n = g.nodes[i]
                inside[v] = body.apply(n.op, [value(x) for x in n.inputs], **n.params)
                return inside[v]
            t = g.types[v]
            inside[v] = body.add_input(t.dtype, t.shape)
            operands.append(v)
            return inside[v]

        member_set = set(members)
        for i in members:
            n = g.nodes[i]
            inside[n.output] = body.apply(n.op, [value(x) for x in n.inputs], **n.params)
        leaving = [g.nodes[i].output for i in members if self.leaves(g.nodes[i].output, member_set)]
        body.set_outputs([inside[v] for v in leaving])
        return body, operands, leaving

    def leaves(self, v: int, member_set: set[int]) -> bool:
        return v in self.outputs or any(u not in member_set for u in self.readers(v))

    # ---- growing groups --------------------------------------------------------------------------------------
    def can_join(self, group: _Group, i: int) -> bool:
        """Node `i` may join `group` when the group still runs before every reader of its values (no reader outside the
        group sits before `i`) and the backend has one kernel for the larger body."""
        member_set = set(group.members)
        for m in group.members:
            for u in self.readers(self.g.nodes[m].output):
                if u < i and u not in member_set:
                    return False
        members = group.members + [i]
        body, _, leaving = self.body_of(members)
        return bool(leaving) and self.accepts(body)

    def run(self) -> G.Graph:
        g = self.g
        if not any(n.op in FUSIBLE for n in g.nodes):
            return g
        self.find_dot_tails()
        in_tail = {i for tail in self.dot_tail.values() for i in tail}
        for i, n in enumerate(g.nodes):
            if n.op == "reshape":
                # a reshape of a group's value (the keepdim of a reduction) runs inside the group; any other is a free view
                p = self.producer.get(n.inputs[0])
                if p is not None and p in self.group_of and i not in in_tail and self.can_join(self.group_of[p], i):
                    self.group_of[p].members.append(i)
                    self.group_of[i] = self.group_of[p]
                continue
            if n.op not in FUSIBLE or i in in_tail:
                continue
            if i in self.transparent:
                continue  # cloned into the groups that read it
            if n.op == "full" and n.output not in self.outputs:
                continue  # a constant some unfusible node reads (the zeros of a scatter-add): stays a plain node
            # the candidate groups: those of the operands' producers, latest first
            candidates = []
            for v in n.inputs:
                for grp in self.source_groups(v):
                    if grp not in candidates:
                        candidates.append(grp)
            candidates.sort(key=lambda grp: -grp.last)
            for grp in candidates:
                if self.can_join(grp, i):
                    grp.members.append(i)
                    self.group_of[i] = grp
                    break
            else:
                grp = _Group(len(self.groups))
                grp.members.append(i)
                self.groups.append(grp)
                self.group_of[i] = grp
        return self.emit()

    # ---- GEMM epilogues ----------------------------------------------------------------------------------------
    def find_dot_tails(self):
        """For each 16-bit `dot_general` read by one node only: the elementwise tail (with its zeros) the GEMM's epilogue
        runs, when the compiler's matcher knows it (relu, `other + product`, `select(0 < other, product, 0)`)."""
        from lumen_b200.compiler import Lowering

        g = self.g
        for i, n in enumerate(g.nodes):
            if n.op != "dot_general" or g.types[n.output].dtype == "float32" or n.output in self.outputs:
                continue
            readers = self.uses.get(n.output, [])
            if len(readers) != 1:
                continue
            tail = readers[0]
            t = g.nodes[tail]
            if t.op not in ("max", "add", "select") or g.types[t.output].shape != g.types[n.output].shape:
                continue
            members = [i, tail]
            if t.op == "select":  # the condition `0 < other` joins too when only the select reads it
                c = self.producer.get(t.inputs[0])
                if c is None or g.nodes[c].op != "lt" or self.uses.get(g.nodes[c].output, []) != [tail]:
                    continue
                members = sorted([i, c, tail])
            # every operand of the tail other than the product has to exist before the dot runs
            outside = [v for m in members for v in g.nodes[m].inputs if self.producer.get(v) not in members]
            if any(self.producer.get(v, -1) > i and g.nodes[self.producer[v]].op not in INLINED for v in outside):
                continue
            body, _, leaving = self.body_of(members)
            if len(leaving) != 1:
                continue
            try:
                Lowering.dot_fusion_epilogue(body)
            except NotImplementedError:
                continue
            self.dot_tail[i] = members

    # ---- rebuilding the graph ------------------------------------------------------------------------------------
    def emit(self) -> G.Graph:
        g = self.g
        out = G.Graph()
        new: dict[int, int] = {}
        for v in g.inputs:
            t = g.types[v]
            new[v] = out.add_input(t.dtype, t.shape)
        emit_at: dict[int, tuple] = {}  # node index of a group's last member -> (members, name, label)
        skipped: set[int] = set()
        for grp in self.groups:
            has_reduce = any(g.nodes[m].op in REDUCTIONS for m in grp.members)
            full_out = False
            if has_reduce:
                _, _, leaving = self.body_of(grp.members)
                rows = max((g.types[g.nodes[m].inputs[0]].numel for m in grp.members if g.nodes[m].op in REDUCTIONS), default=0)
                full_out = any(g.types[v].numel == rows and rows > 0 for v in leaving)
            name = "elementwise" if not has_reduce else ("row" if full_out else "reduction")
            emit_at[grp.last] = (grp.members, name, name)
            skipped.update(grp.members)
        for members in self.dot_tail.values():
            emit_at[members[-1]] = (members, "dot_general", "dot_general_epilogue")
            skipped.update(members)
        dropped = self.transparent
        for i, n in enumerate(g.nodes):
            if i in emit_at:
                members, name, label = emit_at[i]
                body, operands, leaving = self.body_of(members)
                first = out.apply("fusion", [new[v] for v in operands], name=name, label=label, body=body)
                new[leaving[0]] = first
                for k, v in enumerate(leaving[1:], start=1):
                    new[v] = G.fusion_output(out, first, k)
                continue
            if i in skipped:
                continue
            if i in dropped:
                continue
            if n.op == "fusion_output":
                new[n.output] = G.fusion_output(out, new[n.inputs[0]], n.params["index"])
                continue
            new[n.output] = out.apply(n.op, [new[v] for v in n.inputs], **n.params)
        out.set_outputs([new[v] for v in g.outputs])
        return out


def fuse(graph: G.Graph, accepts=_backend_accepts) -> G.Graph:
    """`graph` with its bare elementwise / reduction prims grouped into `fusion` nodes."""
    return FusionPass(graph, accepts).run()
