"""CPU execution of a whole memgraph on the host cores -- TEST INFRASTRUCTURE and the timed CPU
baseline, never part of the product path (only tests/, bench.py's reference / cpu_baseline legs and
the fixture generators import it).

It restates how the reference's CPU server runs a memgraph
(cpu_mg_server_t::execute_memgraph, src/server/cpu/mg_server.cc:13-63; exec nodes
src/engine/cpu/mg/exec_graph.cc:193-318): every node in the memgraph's own order on one big
buffer per location, kernels with the CPU executor's conventions
(src/engine/cpu/kernel_executor.cc) --
  * contractions as permute -> GEMM -> permute with beta = 0 (contraction.cc:103-177,
    kernel_executor.cc:1293-1548): here one torch einsum on the host cores, whose MKL sgemm is
    the closest stand-in available for the cblas_sgemm the reference calls (MKL itself is not
    installed, and the reference's executor source does not compile: merge-conflict markers at
    kernel_executor.cc:1323-1445);
  * elementwise joins with the index conventions of the _unary/_binary/_ternary_ew_loop family
    (kernel_executor.cc:786-914), evaluated from the scalarop tree: f16 inputs, f32 math, one
    rounding at the end (the reference's CPU drivers run f32 because MKL has no f16 kernels,
    llama/first_token.cc:21);
  * reductions with an f64 running total for add / mul and native compares for min / max
    (_real_reduction_ab_a, kernel_executor.cc:1163-1253);
  * touches as engine/touch.cc:155-237 (copy, or += *= min max in the tensor's dtype), fills as
    kernel_executor.cc:1776-1866, moves as byte copies.
The reference runs one kernel per pooled thread (as many threads as cores) and so overlaps
independent nodes; here the nodes run one after the other and every kernel uses all the cores
(torch intra-op threads), which on a mostly sequential layer graph is the faster of the two.

accumulate="f64": contractions accumulate in f64 from the input values and round once -- the
full-size oracle the GPU results are held to (tests/golden/make_c4_full.py).
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import es_oracle as O  # noqa: E402

TD = {"f16": torch.float16, "f32": torch.float32, "f64": torch.float64, "c64": torch.complex64}
SIZE = {"f16": 2, "f32": 4, "f64": 8, "c64": 8}
_CMP = {"<": torch.lt, ">": torch.gt, "==": torch.eq, "<=": torch.le, ">=": torch.ge}


def _compute_dtype(d):
    return torch.float32 if d == "f16" else TD[d]


def eval_tree(node, inputs):
    """The scalarop tree over torch tensors: f16 nodes are computed in f32, convert nodes round."""
    def ev(n):
        t = _compute_dtype(n.dtype)
        if n.op == "constant":
            v = n.value
            if n.dtype == "f16":
                v = float(np.float16(v))
            return torch.tensor(v, dtype=t)
        if n.op == "hole":
            return inputs[n.arg].to(t)
        k = [ev(c) for c in n.kids]
        if n.op == "add":
            return (k[0] + k[1]).to(t)
        if n.op == "mul":
            return (k[0] * k[1]).to(t)
        if n.op == "exp":
            return torch.exp(k[0]).to(t)
        if n.op == "log":
            return torch.log(k[0]).to(t)
        if n.op == "power":
            p = n.power
            if p == 2.0:
                return (k[0] * k[0]).to(t)
            if p == -1.0:
                return torch.reciprocal(k[0]).to(t)
            if p == -0.5:
                return torch.rsqrt(k[0]).to(t)
            if p == 0.5:
                return torch.sqrt(k[0]).to(t)
            return torch.pow(k[0], p).to(t)
        if n.op == "ite":
            return torch.where(_CMP[n.cmp](k[0], k[1]), k[2], k[3]).to(t)
        if n.op == "convert":
            return k[0].to(TD[n.dtype]).to(t)
        if n.op == "conj":
            return torch.conj(k[0]).resolve_conj()
        if n.op == "real":
            return torch.real(k[0]).to(t)
        if n.op == "imag":
            return torch.imag(k[0]).to(t)
        if n.op == "complex":
            return torch.complex(k[0].float(), k[1].float())
        raise ValueError("unknown op " + n.op)

    return ev(node)


def _letters(modes):
    return "".join(chr(ord("a") + m) for m in modes)


class cpu_engine_t:
    def __init__(self, mg, accumulate="f32", threads=None):
        self.mg = mg
        self.accumulate = accumulate
        if threads is None:
            threads = os.cpu_count() or 1
        # torchrun exports OMP_NUM_THREADS=1 to its workers: the thread count is set explicitly
        torch.set_num_threads(int(threads))
        self.threads = torch.get_num_threads()
        self.buffers = [torch.zeros(int(s) + 256, dtype=torch.uint8) for s in mg["mem_sizes"]]
        self.program = []
        self.flops = 0.0
        for node in mg["nodes"]:
            fn = self._compile(node)
            if fn is not None:
                self.program.append(fn)

    # ------------------------------------------------------------------ memory
    def view(self, loc, offset, nelem, dtype, shape=None):
        b = self.buffers[loc][int(offset):int(offset) + int(nelem) * SIZE[dtype]].view(TD[dtype])
        return b.view(list(shape)) if shape is not None else b

    def set_input(self, key, array):
        t = next(x for x in self.mg["inputs"] if x["name"] == key or x["gid"] == key)
        a = np.ascontiguousarray(array, dtype=O.NP_DTYPE[t["dtype"]]).reshape(t["shape"])
        for blk, sl in zip(t["blocks"], O.memgraph_blocks(t["shape"], t["partdims"])):
            raw = np.ascontiguousarray(a[sl]).view(np.uint8).reshape(-1)
            self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]].copy_(torch.from_numpy(raw))

    def get_output(self, key):
        t = next(x for x in self.mg["outputs"] if x["name"] == key or x["gid"] == key)
        out = np.zeros(t["shape"], dtype=O.NP_DTYPE[t["dtype"]])
        for blk, sl in zip(t["blocks"], O.memgraph_blocks(t["shape"], t["partdims"])):
            raw = self.buffers[blk["loc"]][blk["offset"]:blk["offset"] + blk["size"]].numpy()
            out[sl] = raw.view(O.NP_DTYPE[t["dtype"]]).reshape(out[sl].shape)
        return out

    # ------------------------------------------------------------------ nodes
    def _compile(self, node):
        kind = node["kind"]
        if kind in ("alloc", "del", "inputmem", "partialize"):
            return None
        if kind == "apply" and "einsummable" in node:
            return self._einsummable(node)
        if kind == "apply":
            return self._touch(node)
        if kind == "constant":
            return self._fill(node)
        if kind == "move":
            s, so, d, do, n = node["src_loc"], node["src_offset"], node["dst_loc"], node["dst_offset"], node["size"]
            return lambda: self.buffers[d][do:do + n].copy_(self.buffers[s][so:so + n])
        if kind == "copy":
            l, so, do, n = node["loc"], node["src_offset"], node["dst_offset"], node["size"]
            return lambda: self.buffers[l][do:do + n].copy_(self.buffers[l][so:so + n])
        raise ValueError("unknown memgraph node kind %r" % kind)

    def _einsummable(self, node):
        e, loc = node["einsummable"], node["loc"]
        js, inns, out_rank, castable = e["join_shape"], e["inns"], e["out_rank"], e["castable"]
        tree = O.parse_scalarop(e["join"])
        hd = O.hole_dtypes(tree)
        out_shape = js[:out_rank]
        out = self.view(loc, node["mems"][0][0], int(np.prod(out_shape)), tree.dtype, out_shape)
        xs = []
        for k, modes in enumerate(inns):
            shp = [js[m] for m in modes]
            xs.append(self.view(loc, node["mems"][1 + k][0], int(np.prod(shp)), hd[k], shp))
        r = len(js)
        is_contraction = (len(inns) == 2 and castable == "add" and tree.op == "mul" and out_rank < r
                          and tree.kids[0].op == "hole" and tree.kids[1].op == "hole"
                          and tree.kids[0].arg == 0 and tree.kids[1].arg == 1)
        if is_contraction:
            self.flops += 2.0 * float(np.prod(js))
            spec = "%s,%s->%s" % (_letters(inns[0]), _letters(inns[1]), _letters(range(out_rank)))
            wide = torch.float64 if (self.accumulate == "f64" and tree.dtype != "c64") else _compute_dtype(tree.dtype)

            def run():
                out.copy_(torch.einsum(spec, xs[0].to(wide), xs[1].to(wide)))
            return run

        def join_views():
            views = []
            for x, modes in zip(xs, inns):
                order = sorted(range(len(modes)), key=lambda i: modes[i])
                full = [1] * r
                for m in modes:
                    full[m] = js[m]
                views.append(x.permute(order).reshape(full) if len(modes) > 1 else x.reshape(full))
            return views

        if out_rank == r:
            def run():
                res = eval_tree(tree, join_views())
                out.copy_(res.expand(js) if list(res.shape) != list(js) else res)
            return run

        agg = list(range(out_rank, r))

        def run():
            val = eval_tree(tree, join_views())
            if list(val.shape) != list(js):
                val = val.expand(js)
            val = val.to(TD[tree.dtype])        # each join value is a value of the output dtype
            if castable == "add":
                res = val.sum(dim=agg, dtype=torch.float64) if tree.dtype != "c64" else val.sum(dim=agg)
            elif castable == "mul":
                res = val.to(torch.float64).prod(dim=agg[0]) if len(agg) == 1 else None
                if res is None:
                    res = val.to(torch.float64).flatten(out_rank).prod(dim=-1)
            elif castable == "max":
                res = val.float().amax(dim=agg)
            elif castable == "min":
                res = val.float().amin(dim=agg)
            else:
                raise ValueError(castable)
            out.copy_(res)
        return run

    def _touch(self, node):
        t, loc = node["touch"], node["loc"]
        sel, dtype = t["selection"], t["dtype"]
        d_inn = [s[0] for s in sel]
        d_out = [s[1] for s in sel]
        out = self.view(loc, node["mems"][0][0], int(np.prod(d_out)), dtype, d_out)
        inn = self.view(loc, node["mems"][1][0], int(np.prod(d_inn)), dtype, d_inn)
        o = out[tuple(slice(s[3], s[3] + s[4]) for s in sel)]
        i = inn[tuple(slice(s[2], s[2] + s[4]) for s in sel)]
        key = (loc, node["group"])
        castable = t["castable"]

        def run():
            first = node["group"] < 0 or key not in self._groups
            if node["group"] >= 0:
                self._groups.add(key)
            if first or castable is None:
                o.copy_(i)
            elif castable == "add":
                o.add_(i)
            elif castable == "mul":
                o.mul_(i)
            elif castable == "max":
                torch.maximum(o, i, out=o)
            elif castable == "min":
                torch.minimum(o, i, out=o)
            else:
                raise ValueError(castable)
        return run

    def _fill(self, node):
        f, loc, off = node["fill"], node["loc"], node["offset"]
        if f["type"] == "constant":
            dt = f["value"]["dtype"]
            v = O._scalar_from_raw(f["value"]["raw"], dt)
            out = self.view(loc, off, f["nelem"], dt)
            return lambda: out.fill_(complex(v) if dt == "c64" else float(v))
        dt = f["lower"]["dtype"]
        lo = float(O._scalar_from_raw(f["lower"]["raw"], dt))
        up = float(O._scalar_from_raw(f["upper"]["raw"], dt))
        nrow, ncol, start = f["nrow"], f["ncol"], f["start"]
        out = self.view(loc, off, nrow * ncol, dt, [nrow, ncol])

        def run():
            i = torch.arange(nrow).unsqueeze(1)
            j = torch.arange(ncol).unsqueeze(0)
            out.copy_(torch.where(i - start >= j, torch.tensor(lo), torch.tensor(up)))
        return run

    def run(self):
        self._groups = set()
        with torch.no_grad():
            for fn in self.program:
                fn()
