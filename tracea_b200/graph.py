"""Graph front end for conv blocks: load a `GraphTopology`, fuse BatchNorm / residual Add / ReLU into the
producing Conv2d's epilogue, fold BatchNorm into weights and bias, and run the fused graph through
`tracea_conv2d`.

Mirrors, for the Conv2d path only (paths relative to the reference project's root):
  * the JSON form of `GraphTopology` / `OperatorTopology` / `EpilogueOp` as serde writes it
    (src/policy/types.rs:29-95, 188-192; src/core/op.rs:69-90; src/core/loader.rs:9-19):
    externally tagged enums, e.g. {"Conv2d": {"op_id": 1, "name": "conv", "n": 1, ...}} and "ReLU";
  * the fusion pass `GraphOptimizer::apply_fusion` (src/core/optimizer.rs:12-159): a Conv2d whose ONLY
    consumer is a Relu (1 producer), a BatchNorm (5 producers: x, gamma, beta, mean, var, in that order) or an
    Elementwise "Add" (2 producers) absorbs it as the next epilogue op, repeatedly; cases pinned by
    tests/fusion_verification.rs:6-170;
  * BatchNorm arithmetic (x - mean) * rsqrt(var + eps) * gamma + beta (src/core/op.rs:80-81). The reference
    applies it per element at run time (src/emitter/metal/utils.rs:56-73); here it is folded once into the
    conv's weights (scale) and bias (shift), so the kernel's epilogue is bias -> residual -> activation.
"""
import copy
import json

_CONV_KEYS = ("n", "c", "h", "w", "k", "r", "s", "stride", "padding")


# --------------------------------------------------------------------------------- operators (plain dicts)
def op_kind(op):
    """Variant name of an externally tagged operator dict: {"Conv2d": {...}} -> "Conv2d"."""
    (kind,) = op.keys()
    return kind


def op_body(op):
    (body,) = op.values()
    return body


def op_id(op):
    return op_body(op)["op_id"]


def epilogue_name(e):
    """EpilogueOp variant name: unit variants serialise as strings, struct variants as one-key dicts."""
    return e if isinstance(e, str) else next(iter(e))


def conv2d(op_id_, name, n, c, h, w, k, r, s, stride, padding, epilogue=None):
    return {"Conv2d": {"op_id": op_id_, "name": name, "n": n, "c": c, "h": h, "w": w, "k": k, "r": r, "s": s,
                       "stride": stride, "padding": padding, "epilogue": list(epilogue or [])}}


def relu(op_id_, name, n):
    return {"Relu": {"op_id": op_id_, "name": name, "n": n}}


def add(op_id_, name, n):
    return {"Elementwise": {"op_id": op_id_, "name": name, "kind": "Add", "n": n}}


def batchnorm(op_id_, name, n, c, h, w, epsilon=1e-5, momentum=0.1):
    return {"BatchNorm": {"op_id": op_id_, "name": name, "n": n, "c": c, "h": h, "w": w, "epsilon": epsilon,
                          "momentum": momentum}}


def input_op(op_id_, name):
    return {"Input": {"op_id": op_id_, "name": name}}


def load_graph(text_or_path):
    """Parse the JSON the reference's ModelLoader::load_json reads (src/core/loader.rs:9-12)."""
    text = text_or_path
    if not text_or_path.lstrip().startswith("{"):
        with open(text_or_path) as f:
            text = f.read()
    g = json.loads(text)
    if "operators" not in g or "dependencies" not in g:
        raise ValueError("Failed to parse JSON: missing field `operators` or `dependencies`")
    return {"operators": g["operators"], "dependencies": [tuple(d) for d in g["dependencies"]]}


def dump_graph(graph):
    return json.dumps({"operators": graph["operators"], "dependencies": [list(d) for d in graph["dependencies"]]},
                      indent=2)


# --------------------------------------------------------------------------------- fusion pass
def fuse(graph):
    """Restatement of GraphOptimizer::apply_fusion for Conv2d producers. Returns a new graph; producers of a
    fused BatchNorm / Add keep feeding the fused conv (side inputs), as in the reference."""
    ops = copy.deepcopy(graph["operators"])
    adj, radj = {}, {}
    for src, dst in graph["dependencies"]:
        adj.setdefault(src, []).append(dst)
        radj.setdefault(dst, []).append(src)
    removed, fused_into = set(), {}

    def representative(i):
        while i in fused_into:
            i = fused_into[i]
        return i

    modified = True
    while modified:
        modified = False
        by_id = {op_id(o): o for o in ops}
        for op in ops:
            oid = op_id(op)
            if oid in removed or op_kind(op) != "Conv2d":
                continue
            consumers = adj.get(oid, [])
            if len(consumers) != 1 or consumers[0] in removed or consumers[0] not in by_id:
                continue
            cid = consumers[0]
            cop = by_id[cid]
            producers = radj.get(cid, [])
            kind = op_kind(cop)
            if kind == "Relu" and len(producers) == 1:
                e = "ReLU"
            elif kind == "BatchNorm" and len(producers) == 5:
                e = {"BatchNorm": {"op_id": cid, "gamma_id": producers[1], "beta_id": producers[2],
                                   "mean_id": producers[3], "var_id": producers[4],
                                   "epsilon": op_body(cop)["epsilon"]}}
            elif kind == "Elementwise" and op_body(cop)["kind"] == "Add" and len(producers) == 2:
                skip = next((p for p in producers if p != oid), None)
                if skip is None:
                    continue
                e = {"ResidualAdd": {"residual_ptr": representative(skip)}}
            else:
                continue
            op_body(op)["epilogue"].append(e)
            removed.add(cid)
            fused_into[cid] = oid
            # the fused conv takes over the consumer's consumers ...
            cc = adj.get(cid, [])
            adj[oid] = list(cc)
            for x in cc:
                radj[x] = [p for p in radj.get(x, []) if p != cid] + [oid]
            # ... and its side inputs (BN parameters, the skip tensor)
            for p in producers:
                if p != oid:
                    adj.setdefault(p, []).append(oid)
                    radj.setdefault(oid, []).append(p)
            modified = True
        ops = [o for o in ops if op_id(o) not in removed]
    deps = []
    for src, dsts in adj.items():
        if src in removed:
            continue
        for dst in dsts:
            if dst not in removed and (src, dst) not in deps:
                deps.append((src, dst))
    return {"operators": ops, "dependencies": deps}


# --------------------------------------------------------------------------------- a ready-made graph
def bottleneck_graph(n, cin, width, h):
    """A ResNet bottleneck block as UNFUSED operators: conv1x1-bn-relu -> conv3x3-bn-relu -> conv1x1-bn -> add(input)
    -> relu (the block shape of src/bin/network_bench.rs:41-247). Op ids: 0 input, 1 / 4 / 7 the convs, 2 / 5 / 8 their
    BatchNorms, 9 the add, 10 the last ReLU; the BatchNorm parameter inputs are numbered from 101 in the order
    gamma, beta, mean, var per BatchNorm. `fuse` turns it into three convs."""
    ops, deps, oid = [input_op(0, "x")], [], [100]

    def bn_params(bn_id):
        for name in ("gamma", "beta", "mean", "var"):
            oid[0] += 1
            ops.append(input_op(oid[0], "%d.%s" % (bn_id, name)))
            deps.append((oid[0], bn_id))

    ops.append(conv2d(1, "c1", n, cin, h, h, width, 1, 1, 1, 0)); deps.append((0, 1))
    ops.append(batchnorm(2, "bn1", n, width, h, h)); deps.append((1, 2)); bn_params(2)
    ops.append(relu(3, "r1", 0)); deps.append((2, 3))
    ops.append(conv2d(4, "c2", n, width, h, h, width, 3, 3, 1, 1)); deps.append((3, 4))
    ops.append(batchnorm(5, "bn2", n, width, h, h)); deps.append((4, 5)); bn_params(5)
    ops.append(relu(6, "r2", 0)); deps.append((5, 6))
    ops.append(conv2d(7, "c3", n, width, h, h, cin, 1, 1, 1, 0)); deps.append((6, 7))
    ops.append(batchnorm(8, "bn3", n, cin, h, h)); deps.append((7, 8)); bn_params(8)
    ops.append(add(9, "add", 0)); deps.append((8, 9)); deps.append((0, 9))
    ops.append(relu(10, "r3", 0)); deps.append((9, 10))
    return {"operators": ops, "dependencies": deps}


# --------------------------------------------------------------------------------- BatchNorm folding
def fold_batchnorm(weight, gamma, beta, mean, var, eps, conv_bias=None):
    """(x*w [+ b] - mean) * rsqrt(var + eps) * gamma + beta  ==  x*(w*scale) + shift, per output channel:
    scale = gamma * rsqrt(var + eps), shift = beta + ((b or 0) - mean) * scale. Computed in fp32."""
    import torch
    scale = gamma.float() * torch.rsqrt(var.float() + eps)
    w = weight.float() * scale.view(-1, 1, 1, 1)
    b0 = conv_bias.float() if conv_bias is not None else torch.zeros_like(mean, dtype=torch.float32)
    shift = beta.float() + (b0 - mean.float()) * scale
    return w, shift


# --------------------------------------------------------------------------------- execution
_KIND_TABLE = {
    (): "identity", ("bias",): "bias", ("relu",): "relu", ("bias", "relu"): "bias+relu",
    ("residual",): "residual", ("residual", "relu"): "residual+relu", ("bias", "residual"): "bias+residual",
    ("bias", "residual", "relu"): "bias+residual+relu",
}


def epilogue_string(epilogue, has_bias):
    """Epilogue op list of a fused conv -> the op string `tracea_b200.ops` understands. BatchNorm (folded) and a
    conv bias both become "bias"; the order must be [BatchNorm][ResidualAdd][ReLU] (what fusion produces for
    conv -> bn -> add -> relu, tests/fusion_verification.rs:110-170)."""
    names = [epilogue_name(e) for e in epilogue]
    order = {"BatchNorm": 0, "BiasAdd": 0, "ResidualAdd": 1, "ReLU": 2}
    for a, b in zip(names, names[1:]):
        if a not in order or b not in order or order[a] >= order[b]:
            raise ValueError("Unsupported epilogue order %r (supported: [BatchNorm|BiasAdd][ResidualAdd][ReLU])" % (names,))
    if len(names) == 1 and names[0] not in order:
        raise ValueError("Unsupported epilogue op %r" % names[0])
    parts = []
    if has_bias or "BatchNorm" in names or "BiasAdd" in names:
        parts.append("bias")
    if "ResidualAdd" in names:
        parts.append("residual")
    if "ReLU" in names:
        parts.append("relu")
    return _KIND_TABLE[tuple(parts)]


class GraphRunner:
    """Runs a FUSED graph whose compute ops are all Conv2d. `params[op_id]` holds, per conv, {"weight": OIHW
    tensor, optional "bias"}; per BatchNorm parameter input op id, a 1-D tensor. `inputs[op_id]` holds the
    tensors of the remaining Input ops (logical NCHW). Everything lives on one CUDA device; tensors are kept
    channels-last so that every conv takes the zero-copy path."""

    def __init__(self, graph, params, dtype=None):
        import torch
        self.graph = graph
        self.ops = {op_id(o): o for o in graph["operators"]}
        self.order = self._topological_order()
        self.plan = []
        self._resident = {}
        for oid in self.order:
            op = self.ops[oid]
            if op_kind(op) == "Input":
                continue
            if op_kind(op) != "Conv2d":
                raise ValueError("operator %r (%s) was not fused into a conv and cannot be executed here"
                                 % (op_body(op)["name"], op_kind(op)))
            b = op_body(op)
            w = params[oid]["weight"]
            bias = params[oid].get("bias")
            for e in b["epilogue"]:
                if epilogue_name(e) == "BatchNorm":
                    bn = e["BatchNorm"]
                    w, bias = fold_batchnorm(w, params[bn["gamma_id"]], params[bn["beta_id"]], params[bn["mean_id"]],
                                             params[bn["var_id"]], bn["epsilon"], bias)
            dt = dtype or params[oid]["weight"].dtype
            w = w.to(dt).contiguous(memory_format=torch.channels_last)
            res_id = next((e["ResidualAdd"]["residual_ptr"] for e in b["epilogue"]
                           if epilogue_name(e) == "ResidualAdd"), None)
            side = {x for e in b["epilogue"] if epilogue_name(e) == "BatchNorm"
                    for x in (e["BatchNorm"][k] for k in ("gamma_id", "beta_id", "mean_id", "var_id"))}
            srcs = [s for s, d in graph["dependencies"] if d == oid and s != res_id and s not in side]
            if len(srcs) != 1:
                raise ValueError("conv %r must have exactly one data input, found %r" % (b["name"], srcs))
            self.plan.append((oid, srcs[0], res_id, w, bias.float() if bias is not None else None,
                              epilogue_string(b["epilogue"], bias is not None), b["stride"], b["padding"]))

    def _topological_order(self):
        indeg = {i: 0 for i in self.ops}
        for s, d in self.graph["dependencies"]:
            if s in self.ops and d in self.ops:
                indeg[d] += 1
        ready = sorted(i for i, n in indeg.items() if n == 0)
        order = []
        while ready:
            i = ready.pop(0)
            order.append(i)
            for s, d in self.graph["dependencies"]:
                if s == i and d in indeg:
                    indeg[d] -= 1
                    if indeg[d] == 0:
                        ready.append(d)
        if len(order) != len(self.ops):
            raise ValueError("graph has a cycle")
        return order

    def run(self, inputs):
        """inputs: {input op id: tensor}. Returns {conv op id: output tensor} for every conv."""
        import torch
        from . import ops
        values = {i: t.contiguous(memory_format=torch.channels_last) for i, t in inputs.items()}
        for oid, src, res_id, w, bias, epi, stride, padding in self.plan:
            x = values[src]
            if not x.is_cuda:
                raise ValueError("GraphRunner inputs must be CUDA tensors")
            res = values[res_id] if res_id is not None else None
            key = (oid, x.device)
            if key not in self._resident:      # folded weights and bias are uploaded once per device
                self._resident[key] = (w.to(x.device), bias.to(x.device) if bias is not None else None)
            dev_w, dev_bias = self._resident[key]
            values[oid] = ops.conv2d_nchw(x, dev_w, dev_bias, res, stride, padding, 1, 1,
                                          None if epi == "identity" else epi, channels_last_out=True)
        return values

    def run_host(self, inputs, outputs, device=None, chunks=8):
        """The same graph for tensors that live in HOST memory: `inputs` {input op id: CPU tensor} are copied to
        the device once, the whole chain of convs runs there, and only the tensors named in `outputs`
        {conv op id: CPU tensor to fill} come back -- intermediates never cross the bus (the reference's executor
        keeps them in its device arena, src/runtime/manager/graph.rs:7-50, src/runtime/executor/mod.rs:79-85).
        A convolution never mixes images, so the batch is cut into `chunks` slices whose copy-in, kernels and
        copy-out overlap on three streams (the bus is full duplex). Pinned host tensors make the copies
        asynchronous; pageable ones work, without the overlap. Returns when `outputs` are filled."""
        import torch
        from . import ops
        dev = torch.device(device if device is not None else "cuda")
        n = next(iter(inputs.values())).shape[0]
        if any(t.shape[0] != n for t in inputs.values()):
            raise ValueError("every input must have the same batch size")
        chunks = max(1, min(chunks, n))
        cl = torch.channels_last
        key = (dev, tuple(sorted((i, tuple(t.shape), t.dtype) for i, t in inputs.items())), tuple(sorted(outputs)))
        st = self._host_state.get(key) if hasattr(self, "_host_state") else None
        if st is None:
            if not hasattr(self, "_host_state"):
                self._host_state = {}
            st = {
                "in": {i: torch.empty(t.shape, dtype=t.dtype, device=dev).contiguous(memory_format=cl)
                       for i, t in inputs.items()},
                "copy_in": torch.cuda.Stream(dev), "copy_out": torch.cuda.Stream(dev),
                "ev_in": [], "ev_done": [],
            }
            self._host_state[key] = st
        while len(st["ev_in"]) < chunks:
            st["ev_in"].append(torch.cuda.Event())
            st["ev_done"].append(torch.cuda.Event())
        main = torch.cuda.current_stream(dev)
        st["copy_in"].wait_stream(main)
        st["copy_out"].wait_stream(main)
        bounds = [(n * c // chunks, n * (c + 1) // chunks) for c in range(chunks)]
        for c, (a, b) in enumerate(bounds):
            with torch.cuda.stream(st["copy_in"]):
                for i, t in inputs.items():
                    st["in"][i][a:b].copy_(t[a:b], non_blocking=True)
                st["ev_in"][c].record(st["copy_in"])
            main.wait_event(st["ev_in"][c])
            values = self.run({i: st["in"][i][a:b] for i in inputs})
            st["ev_done"][c].record(main)
            with torch.cuda.stream(st["copy_out"]):
                st["copy_out"].wait_event(st["ev_done"][c])
                for oid, host in outputs.items():
                    values[oid].record_stream(st["copy_out"])
                    host[a:b].copy_(values[oid], non_blocking=True)
        main.wait_stream(st["copy_out"])
        main.synchronize()
        return outputs
