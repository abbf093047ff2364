"""The attention passes: find `softmax(score_ops(Q K^T)) V` - and the FlashAttention-2 backward traced from it - in a
graph of bare prims and rewrite each into ONE fusion (`flash_attention` / `flash_attention_backward`) that the backend
runs as its tcgen05 kernels.

Counterpart of the reference's passes (lumen/graph_compiler/passes/attention/forward.rs:56-97,598-772 and
backward.rs:54-83,238-525). As there, the match starts from the product with the values and walks up:

    o   = dot_general(p, v)                     float32 accumulation, [B, N, Sq, Hv]
    p   = cast(e / broadcast(sum(e)))           probabilities, rounded to the operands' dtype before the product
    e   = exp(s - broadcast(max(s)))
    s   = select(key <= query + c, s', -inf)    optional causal mask from two iotas
    s'  = dot_general(q, k) * scale             optional positive constant scale; float32 scores, [B, N, Sq, Sk]

plus, when the program computes it, the row log-sum-exp `max + log(sum)` as a second output. Operands may reach the
products through transposes (a `[B, S, N, H]` tensor permuted to `[B, N, S, H]`) and through the grouped-query head
expansion (`reshape -> broadcast -> reshape` of `[B, S, Nkv, H]`); the output may be permuted back to `[B, S, N, H]`.
The fusion's BODY is the matched subgraph itself, node for node, so evaluating the rewritten graph primitive by
primitive gives exactly what the original gives (the reference requires the same of every pass,
lumen/reference/README.md:15). What the kernel needs - which dimension of each source tensor is batch, sequence, head
and head dim, the scale, the mask offset - is attached to the fusion node as `attention=` parameters.

The backward matcher is keyed, like the reference's, on the recomputed transposed probabilities `exp(s^T - lse)`: it
recognises the backward `lumen_b200.functional.attention_backward_prims` traces (lumen/functional/attention/flash.py:
51-85), the one spelling autograd produces.
"""

from __future__ import annotations

import math

from lumen_b200 import graph as G


class Match(Exception):
    """Raised inside a matcher when the subgraph at hand is not the pattern."""


def _need(cond, why=""):
    if not cond:
        raise Match(why)


class Rewriter:
    def __init__(self, graph: G.Graph):
        self.g = graph
        self.index()

    def index(self):
        g = self.g
        self.prod = {n.output: i for i, n in enumerate(g.nodes)}
        self.users: dict[int, list[int]] = {}
        for i, n in enumerate(g.nodes):
            for v in n.inputs:
                self.users.setdefault(v, []).append(i)
        # Nodes the fusion body may hold a COPY of while other readers keep the original: values that depend on no
        # input (masks from iotas, constants: common-subexpression elimination shares them between the forward and the
        # backward) and pure re-layouts (transposes, the reshape / broadcast of the head expansion).
        self.input_free = set()
        for i, n in enumerate(g.nodes):
            if n.op in ("full", "iota") or (n.inputs and n.op not in ("fusion", "fusion_output") and all(self.prod.get(v) in self.input_free for v in n.inputs)):
                self.input_free.add(i)

    def shareable(self, i):
        return i in self.input_free or self.g.nodes[i].op in ("transpose", "reshape", "broadcast_in_dim")

    # ---- small helpers --------------------------------------------------------------------------------------------
    def node(self, v):
        i = self.prod.get(v)
        return None if i is None else self.g.nodes[i]

    def is_op(self, v, op):
        n = self.node(v)
        return n is not None and n.op == op

    def constant(self, v):
        """The Python value of a (possibly broadcast) scalar `full`, else None."""
        n = self.node(v)
        if n is not None and n.op == "broadcast_in_dim":
            n = self.node(n.inputs[0])
        if n is not None and n.op == "full" and self.g.types[n.output].shape == ():
            return n.params["fill_value"]
        return None

    def keepdim_of(self, v, reduce_op, last_axis):
        """`v` = a row reduction of something over `last_axis`, broadcast back to the full shape (through the `[.., 1]`
        reshape a keepdim makes, or directly). Returns (reduced operand, reduction node index, the `[.., 1]` value or
        None, every node index in between)."""
        n = self.node(v)
        _need(n is not None and n.op == "broadcast_in_dim")
        inner, used, keep = n.inputs[0], [self.prod[v]], None
        m = self.node(inner)
        if m is not None and m.op == "reshape" and self.g.types[inner].shape[-1:] == (1,):
            keep = inner
            used.append(self.prod[inner])
            inner = m.inputs[0]
            m = self.node(inner)
            _need(tuple(n.params["broadcast_dimensions"]) == tuple(range(last_axis + 1)))
        else:
            _need(tuple(n.params["broadcast_dimensions"]) == tuple(range(last_axis)))
        _need(m is not None and m.op == reduce_op and tuple(m.params["axes"]) == (last_axis,))
        used.append(self.prod[inner])
        return m.inputs[0], self.prod[inner], keep, used

    def source(self, v, roles):
        """Walks from a product's operand `v` (its dimensions labelled by `roles`, e.g. "BNSH") up through transposes and
        the grouped-query head expansion to the tensor the kernel will read. Returns (source value, roles of the
        source's dimensions, heads per key/value head, node indices walked through)."""
        used, group = [], 1
        while True:
            n = self.node(v)
            if n is not None and n.op == "transpose":
                perm = n.params["permutation"]
                # output dim d is input dim perm[d]
                inner = [None] * len(perm)
                for d, p in enumerate(perm):
                    inner[p] = roles[d]
                roles = "".join(inner)
                used.append(self.prod[v])
                v = n.inputs[0]
                continue
            if n is not None and n.op == "reshape" and group == 1:
                # [.., Nkv, 1, ..] -> broadcast -> [.., Nkv, G, ..] -> reshape [.., N, ..]
                b = self.node(n.inputs[0])
                if b is not None and b.op == "broadcast_in_dim":
                    r = self.node(b.inputs[0])
                    wide, mid = self.g.types[b.output].shape, self.g.types[b.inputs[0]].shape
                    out = self.g.types[v].shape
                    if r is not None and r.op == "reshape" and len(wide) == len(out) + 1 == len(mid):
                        at = roles.index("N")
                        src_shape = self.g.types[r.inputs[0]].shape
                        ok = (len(src_shape) == len(out) and mid[at + 1] == 1 and mid[:at + 1] == src_shape[:at + 1]
                              and mid[at + 2:] == src_shape[at + 1:] and wide[:at + 1] == mid[:at + 1] and wide[at + 2:] == mid[at + 2:]
                              and out[at] == wide[at] * wide[at + 1] and out[:at] == wide[:at] and out[at + 1:] == wide[at + 2:]
                              and tuple(b.params["broadcast_dimensions"]) == tuple(range(len(wide))))
                        if ok:
                            group = wide[at + 1]
                            used += [self.prod[v], self.prod[n.inputs[0]], self.prod[b.inputs[0]]]
                            v = r.inputs[0]
                            continue
            return v, roles, group, used

    # ---- forward ---------------------------------------------------------------------------------------------------
    def match_forward(self, pv_index):
        g = self.g
        pv = g.nodes[pv_index]
        _need(pv.op == "dot_general")
        p_v, v_v = pv.inputs
        pt = g.types[p_v]
        _need(len(pt.shape) == 4 and tuple(pv.params["lhs_batch"]) == (0, 1) and tuple(pv.params["lhs_contracting"]) == (3,))
        _need(pv.params["accum_dtype"] == "float32")
        rb, rc = tuple(pv.params["rhs_batch"]), tuple(pv.params["rhs_contracting"])
        _need(len(rb) == 2 and len(rc) == 1 and len(g.types[v_v].shape) == 4)
        v_roles = [None] * 4
        v_roles[rb[0]], v_roles[rb[1]], v_roles[rc[0]] = "B", "N", "S"
        v_roles[v_roles.index(None)] = "H"
        used = [pv_index]
        # p = cast(e / broadcast(sum(e))) in the operands' dtype
        dtype = g.types[v_v].dtype
        n = self.node(p_v)
        _need(n is not None)
        if n.op == "cast":
            _need(g.types[p_v].dtype == dtype)
            used.append(self.prod[p_v])
            n = self.node(n.inputs[0])
        _need(n is not None and n.op == "div" and g.types[n.output].dtype == "float32")
        used.append(self.prod[n.output])
        e_v, total_b = n.inputs
        summed, sum_index, total_keep, walked = self.keepdim_of(total_b, "reduce_sum", 3)
        _need(summed == e_v and g.nodes[sum_index].params["accum_dtype"] == "float32")
        used += walked
        e = self.node(e_v)
        _need(e is not None and e.op == "exp")
        used.append(self.prod[e_v])
        sub = self.node(e.inputs[0])
        _need(sub is not None and sub.op == "sub")
        used.append(self.prod[sub.output])
        s_v, max_b = sub.inputs
        maxed, _, max_keep, walked = self.keepdim_of(max_b, "reduce_max", 3)
        _need(maxed == s_v)
        used += walked
        # optional causal mask: select(key <= query + c, s', -inf)
        causal, offset = False, 0
        n = self.node(s_v)
        if n is not None and n.op == "select":
            cond, kept, fill = n.inputs
            _need(self.constant(fill) == float("-inf"))
            offset, walked = self.match_causal(cond)
            causal = True
            used += [self.prod[s_v], *walked] + self.constant_nodes(fill)
            s_v = kept
            n = self.node(s_v)
        # optional scale: dot * positive constant
        scale = 1.0
        if n is not None and n.op == "mul":
            a, b = n.inputs
            c = self.constant(b)
            if c is None:
                a, b = b, a
                c = self.constant(b)
            _need(c is not None and float(c) > 0.0, "scores scaled by something other than a positive constant")
            scale = float(c)
            used += [self.prod[s_v]] + self.constant_nodes(b)
            s_v = a
            n = self.node(s_v)
        _need(n is not None and n.op == "dot_general" and g.types[s_v].dtype == "float32" and n.params["accum_dtype"] == "float32")
        used.append(self.prod[s_v])
        q_v, k_v = n.inputs
        lb, lc = tuple(n.params["lhs_batch"]), tuple(n.params["lhs_contracting"])
        kb, kc = tuple(n.params["rhs_batch"]), tuple(n.params["rhs_contracting"])
        _need(len(lb) == 2 and len(lc) == 1 and len(kb) == 2 and len(kc) == 1 and len(g.types[q_v].shape) == 4 and len(g.types[k_v].shape) == 4)
        q_roles, k_roles = [None] * 4, [None] * 4
        q_roles[lb[0]], q_roles[lb[1]], q_roles[lc[0]] = "B", "N", "H"
        q_roles[q_roles.index(None)] = "S"
        k_roles[kb[0]], k_roles[kb[1]], k_roles[kc[0]] = "B", "N", "H"
        k_roles[k_roles.index(None)] = "S"
        _need(g.types[q_v].dtype == dtype and g.types[k_v].dtype == dtype)
        sources = {}
        for name, value, roles in (("q", q_v, q_roles), ("k", k_v, k_roles), ("v", v_v, v_roles)):
            src, src_roles, group, walked = self.source(value, "".join(roles))
            sources[name] = (src, src_roles, group)
            used += walked
        _need(sources["k"][2] == sources["v"][2], "keys and values expand their heads differently")
        # the output: the product, its cast to the operands' dtype, and a permutation back to [B, S, N, H] when it is the only use
        out_v, out_roles = pv.output, "BNSH"
        if g.types[out_v].dtype != dtype:
            us = self.users.get(out_v, [])
            _need(len(us) == 1 and g.nodes[us[0]].op == "cast" and g.types[g.nodes[us[0]].output].dtype == dtype and out_v not in g.outputs)
            used.append(us[0])
            out_v = g.nodes[us[0]].output
        us = self.users.get(out_v, [])
        if len(us) == 1 and g.nodes[us[0]].op == "transpose" and out_v not in g.outputs:
            perm = g.nodes[us[0]].params["permutation"]
            out_roles = "".join(out_roles[p] for p in perm)
            used.append(us[0])
            out_v = g.nodes[us[0]].output
        # the log-sum-exp, if the program computes it: max + log(sum) on the keepdim values
        lse_v = None
        if max_keep is not None and total_keep is not None:
            for u in self.users.get(total_keep, []):
                ln = g.nodes[u]
                if ln.op != "log":
                    continue
                for u2 in self.users.get(ln.output, []):
                    add = g.nodes[u2]
                    if add.op == "add" and set(add.inputs) == {max_keep, ln.output}:
                        lse_v = add.output
                        used += [u, u2]
        used = sorted(set(used))
        outputs = [out_v] + ([lse_v] if lse_v is not None else [])
        inside = {g.nodes[i].output for i in used}
        for i in used:  # nothing computed inside may be read from outside (the probabilities are never materialised)
            v = g.nodes[i].output
            if v in outputs or self.shareable(i):
                continue
            _need(v not in g.outputs and all(u in used for u in self.users.get(v, [])), "an inner value of the attention is used elsewhere")
        info = {"scale": scale, "causal": causal, "offset": int(offset), "heads_per_kv": sources["k"][2],
                "q": sources["q"][1], "k": sources["k"][1], "v": sources["v"][1], "o": out_roles, "lse": lse_v is not None}
        operands = [sources["q"][0], sources["k"][0], sources["v"][0]]
        _need(all(v not in inside for v in operands))
        return used, operands, outputs, info

    def constant_nodes(self, v):
        out = []
        n = self.node(v)
        if n is not None and n.op == "broadcast_in_dim":
            out.append(self.prod[v])
            v = n.inputs[0]
            n = self.node(v)
        if n is not None and n.op == "full":
            out.append(self.prod[v])
        return out

    def match_causal(self, cond, key_dim=3, query_dim=2):
        """`key <= query + c` as the tracer spells `<=`: select(lt, lt, eq) over iota(key_dim) and iota(query_dim) + c.
        Returns (c, node indices)."""
        n = self.node(cond)
        _need(n is not None and n.op == "select" and n.inputs[0] == n.inputs[1])
        lt, eq = self.node(n.inputs[0]), self.node(n.inputs[2])
        _need(lt is not None and eq is not None and lt.op == "lt" and eq.op == "eq" and tuple(lt.inputs) == tuple(eq.inputs))
        keys, bound = lt.inputs
        kn = self.node(keys)
        _need(kn is not None and kn.op == "iota" and kn.params["dimension"] == key_dim)
        used = [self.prod[cond], self.prod[lt.output], self.prod[eq.output], self.prod[keys]]
        offset = 0
        bn = self.node(bound)
        if bn is not None and bn.op == "add":
            a, b = bn.inputs
            c = self.constant(b)
            if c is None:
                a, b = b, a
                c = self.constant(b)
            _need(c is not None and isinstance(c, int))
            offset = int(c)
            used += [self.prod[bound]] + self.constant_nodes(b)
            bound = a
            bn = self.node(bound)
        _need(bn is not None and bn.op == "iota" and bn.params["dimension"] == query_dim)
        used.append(self.prod[bound])
        return offset, used

    # ---- backward --------------------------------------------------------------------------------------------------
    def match_backward(self, exp_index):
        """Keyed on `pt = exp(st - broadcast(lse))` with `st` the transposed scores `dot_general(k, q)` (scaled, masked):
        the program `attention_backward_prims` traces, piece by piece -

            dst = cast(pt * (dot(v, dO) - delta) * scale),   delta = rowsum(dO * O) as a batch-only dot_general
            dV = dot(cast(pt), dO),  dK = dot(dst, q),  dQ = dot(dst, k)

        each gradient permuted back to `[B, S, N, H]`, summed over the query heads of a key/value head when heads are
        grouped, and cast to the operands' dtype. Operands: q, k, v, o, lse, dO, all `[B, S, N, H]` (lse `[B, N, Sq, 1]`)."""
        g = self.g
        e = g.nodes[exp_index]
        _need(e.op == "exp")
        sub = self.node(e.inputs[0])
        _need(sub is not None and sub.op == "sub")
        st_v, lse_b = sub.inputs
        bn = self.node(lse_b)
        _need(bn is not None and bn.op == "broadcast_in_dim" and tuple(bn.params["broadcast_dimensions"]) == (0, 1, 2, 3))
        lse_r = self.node(bn.inputs[0])
        _need(lse_r is not None and lse_r.op == "reshape" and g.types[lse_r.output].shape[2] == 1)
        lse_src = lse_r.inputs[0]
        used = [exp_index, self.prod[sub.output], self.prod[lse_b], self.prod[lse_r.output]]
        causal, offset, scale = False, 0, 1.0
        n = self.node(st_v)
        if n is not None and n.op == "select":
            cond, kept, fill = n.inputs
            _need(self.constant(fill) == float("-inf"))
            offset, walked = self.match_causal_transposed(cond)
            causal = True
            used += [self.prod[st_v], *walked] + self.constant_nodes(fill)
            st_v = kept
            n = self.node(st_v)
        if n is not None and n.op == "mul":
            st_v, c, walked = self.times_constant(n)
            scale = c
            used += walked
            n = self.node(st_v)
        _need(n is not None and n.op == "dot_general" and n.params["accum_dtype"] == "float32")
        _need(tuple(n.params["lhs_batch"]) == (0, 2) and tuple(n.params["rhs_batch"]) == (0, 2)
              and tuple(n.params["lhs_contracting"]) == (3,) and tuple(n.params["rhs_contracting"]) == (3,))
        used.append(self.prod[st_v])
        ke_v, q_v = n.inputs
        dtype = g.types[q_v].dtype
        k_src, k_roles, group, walked = self.source(ke_v, "BSNH")
        _need(k_roles == "BSNH")
        used += walked
        # the two readers of pt: its cast (for dV) and the product with (dpt - delta)
        pt_users = self.users.get(e.output, [])
        _need(len(pt_users) == 2 and e.output not in g.outputs)
        cast_i = next((u for u in pt_users if g.nodes[u].op == "cast"), None)
        mul_i = next((u for u in pt_users if g.nodes[u].op == "mul"), None)
        _need(cast_i is not None and mul_i is not None and g.types[g.nodes[cast_i].output].dtype == dtype)
        used += [cast_i, mul_i]
        other = [v for v in g.nodes[mul_i].inputs if v != e.output]
        _need(len(other) == 1)
        diff = self.node(other[0])
        _need(diff is not None and diff.op == "sub")
        used.append(self.prod[other[0]])
        dpt_v, delta_b = diff.inputs
        dpt = self.node(dpt_v)
        _need(dpt is not None and dpt.op == "dot_general" and tuple(dpt.params["lhs_batch"]) == (0, 2) and tuple(dpt.params["rhs_batch"]) == (0, 2)
              and tuple(dpt.params["lhs_contracting"]) == (3,) and tuple(dpt.params["rhs_contracting"]) == (3,))
        used.append(self.prod[dpt_v])
        ve_v, do_v = dpt.inputs
        v_src, v_roles, v_group, walked = self.source(ve_v, "BSNH")
        _need(v_roles == "BSNH" and v_group == group)
        used += walked
        # delta: broadcast(reshape(transpose(dot(dO, O) over the head dim, batch (0, 1, 2))))
        dn = self.node(delta_b)
        _need(dn is not None and dn.op == "broadcast_in_dim")
        used.append(self.prod[delta_b])
        x = dn.inputs[0]
        for op in ("reshape", "transpose"):
            xn = self.node(x)
            _need(xn is not None and xn.op == op)
            used.append(self.prod[x])
            x = xn.inputs[0]
        dd = self.node(x)
        _need(dd is not None and dd.op == "dot_general" and tuple(dd.params["lhs_batch"]) == (0, 1, 2) and tuple(dd.params["lhs_contracting"]) == (3,))
        used.append(self.prod[x])
        _need(dd.inputs[0] == do_v)
        o_v = dd.inputs[1]
        # dst = cast(pt * (dpt - delta) * scale)
        v = g.nodes[mul_i].output
        us = self.users.get(v, [])
        _need(len(us) == 1)
        nxt = g.nodes[us[0]]
        if nxt.op == "mul":
            _, c2, walked = self.times_constant(nxt)
            _need(abs(c2 - scale) <= 1e-12 * scale, "the backward scales dS by another constant than the scores")
            used += walked
            v = nxt.output
            us = self.users.get(v, [])
            _need(len(us) == 1)
            nxt = g.nodes[us[0]]
        else:
            _need(scale == 1.0)
        _need(nxt.op == "cast" and g.types[nxt.output].dtype == dtype)
        used.append(us[0])
        dst_v = nxt.output
        # the three products and what follows each up to the gradient
        dst_users = self.users.get(dst_v, [])
        _need(len(dst_users) == 2 and all(g.nodes[u].op == "dot_general" for u in dst_users))
        dq_i = next((u for u in dst_users if tuple(g.nodes[u].params["lhs_contracting"]) == (2,)), None)
        dk_i = next((u for u in dst_users if tuple(g.nodes[u].params["lhs_contracting"]) == (3,)), None)
        _need(dq_i is not None and dk_i is not None and g.nodes[dq_i].inputs[1] == ke_v and g.nodes[dk_i].inputs[1] == q_v)
        ptc_users = self.users.get(g.nodes[cast_i].output, [])
        _need(len(ptc_users) == 1 and g.nodes[ptc_users[0]].op == "dot_general" and g.nodes[ptc_users[0]].inputs[1] == do_v)
        dv_i = ptc_users[0]
        outputs = []
        for i in (dq_i, dk_i, dv_i):
            used.append(i)
            v = g.nodes[i].output
            while g.types[v].dtype != dtype or (len(self.users.get(v, [])) == 1 and v not in g.outputs
                                              and g.nodes[self.users[v][0]].op in ("transpose", "reshape", "reduce_sum", "cast")):
                us = self.users.get(v, [])
                _need(len(us) == 1 and g.nodes[us[0]].op in ("transpose", "reshape", "reduce_sum", "cast") and v not in g.outputs)
                used.append(us[0])
                v = g.nodes[us[0]].output
            outputs.append(v)
        used = sorted(set(used))
        inside = {g.nodes[i].output for i in used}
        for i in used:
            v = g.nodes[i].output
            if v in outputs or self.shareable(i):
                continue
            _need(v not in g.outputs and all(u in used for u in self.users.get(v, [])), "an inner value of the attention backward is used elsewhere")
        operands = [q_v, k_src, v_src, o_v, lse_src, do_v]
        _need(all(v not in inside for v in operands))
        for name, v in zip(("dq", "dk", "dv"), outputs):
            want = g.types[q_v if name == "dq" else (k_src if name == "dk" else v_src)].shape
            _need(g.types[v].shape == want, f"{name} does not have its operand's shape")
        info = {"scale": scale, "causal": causal, "offset": int(offset), "heads_per_kv": group}
        return used, operands, outputs, info

    def times_constant(self, n):
        """`n` = mul(x, positive constant) in either order: (x, constant, node indices)."""
        a, b = n.inputs
        c = self.constant(b)
        if c is None:
            a, b = b, a
            c = self.constant(b)
        _need(c is not None and float(c) > 0.0, "scaled by something other than a positive constant")
        return a, float(c), [self.prod[n.output]] + self.constant_nodes(b)

    def match_causal_transposed(self, cond):
        """The mask of the transposed scores `[B, N, Sk, Sq]`: key (dim 2) <= query (dim 3) + c."""
        return self.match_causal(cond, key_dim=2, query_dim=3)

    # ---- rewriting -------------------------------------------------------------------------------------------------
    def fuse(self, members, operands, outputs, name, info):
        """Replaces the nodes `members` by one fusion node (plus `fusion_output`s) whose body is those nodes."""
        g = self.g
        body = G.Graph()
        inside = {}
        for v in operands:
            t = g.types[v]
            inside[v] = body.add_input(t.dtype, t.shape)
        for i in members:
            n = g.nodes[i]
            for v in n.inputs:
                if v not in inside:
                    raise Match(f"value %{v} enters the matched region but is not one of its operands")
            inside[n.output] = body.apply(n.op, [inside[v] for v in n.inputs], **n.params)
        body.set_outputs([inside[v] for v in outputs])
        member_set = set(members)
        # a shared member (a constant, a re-layout) that something outside still reads stays in the graph as well
        stays = {i for i in members if g.nodes[i].output not in outputs
                 and (g.nodes[i].output in g.outputs or any(u not in member_set for u in self.users.get(g.nodes[i].output, [])))}
        changed = True
        while changed:  # and so does whatever such a node reads from inside
            changed = False
            for i in list(stays):
                for v in g.nodes[i].inputs:
                    p = self.prod.get(v)
                    if p in member_set and p not in stays:
                        stays.add(p)
                        changed = True
        last = max(members)
        new_nodes = []
        for i, n in enumerate(g.nodes):
            if i == last:
                params = {"body": body, "name": name, "label": name, "attention": info}
                new_nodes.append(G.Node("fusion", tuple(operands), outputs[0], params))
                for k, v in enumerate(outputs[1:], start=1):
                    new_nodes.append(G.Node("fusion_output", (outputs[0],), v, {"index": k}))
            if i not in member_set or i in stays:
                new_nodes.append(n)
        # a reader of an output that sat between the region's nodes must come after the fusion: keep program order valid
        g.nodes = self.reorder(new_nodes)
        self.index()

    def reorder(self, nodes):
        """Stable topological order (values are defined before they are read)."""
        defined = set(self.g.inputs)
        pending, out = list(nodes), []
        while pending:
            progressed = False
            rest = []
            for n in pending:
                if all(v in defined for v in n.inputs):
                    out.append(n)
                    defined.add(n.output)
                    progressed = True
                else:
                    rest.append(n)
            if not progressed:
                raise Match("the rewritten graph has a cycle")
            pending = rest
        return out

    def run(self):
        changed = True
        while changed:
            changed = False
            for i, n in enumerate(self.g.nodes):
                if n.op == "dot_general":
                    try:
                        found = self.match_forward(i)
                    except Match:
                        continue
                    try:
                        self.fuse(found[0], found[1], found[2], "flash_attention", found[3])
                    except Match:
                        continue
                    changed = True
                    break
                if n.op == "exp":
                    try:
                        members, operands, outputs, info = self.match_backward(i)
                        self.fuse(members, operands, outputs, "flash_attention_backward", info)
                    except Match:
                        continue
                    changed = True
                    break
        return self.g


def match_attention(graph: G.Graph) -> G.Graph:
    """`graph` with every attention forward / backward written in bare prims replaced by a `flash_attention` /
    `flash_attention_backward` fusion (a rewritten copy). Graphs without the pattern pass through unchanged."""
    if not any(n.op == "dot_general" for n in graph.nodes):
        return graph
    work = G.Graph()  # the caller's graph is left as traced
    work.types, work.inputs, work.outputs, work.nodes = list(graph.types), list(graph.inputs), list(graph.outputs), list(graph.nodes)
    return Rewriter(work).run()


_ = math
