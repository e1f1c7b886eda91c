"""The graph front end: fusion of Conv+BN+Add+ReLU into a conv epilogue and BatchNorm folding.
The first three cases are the ones the reference pins in tests/fusion_verification.rs:6-170."""
import json

import pytest
import torch
import torch.nn.functional as F

from tracea_b200 import graph as G


def _find(graph, oid):
    return next(o for o in graph["operators"] if G.op_id(o) == oid)


def test_conv_relu_fusion():
    g = {"operators": [G.conv2d(1, "conv", 1, 3, 224, 224, 64, 3, 3, 1, 1), G.relu(2, "relu", 64 * 224 * 224)],
         "dependencies": [(1, 2)]}
    f = G.fuse(g)
    assert len(f["operators"]) == 1
    assert G.op_body(f["operators"][0])["epilogue"] == ["ReLU"]
    assert len(g["operators"]) == 2 and G.op_body(g["operators"][0])["epilogue"] == []   # input graph untouched


def test_conv_bn_relu_fusion():
    ops = [G.conv2d(1, "conv", 1, 3, 224, 224, 64, 3, 3, 1, 1), G.batchnorm(2, "bn", 1, 64, 224, 224),
           G.relu(3, "relu", 64 * 224 * 224), G.input_op(10, "gamma"), G.input_op(11, "beta"),
           G.input_op(12, "mean"), G.input_op(13, "var")]
    deps = [(1, 2), (10, 2), (11, 2), (12, 2), (13, 2), (2, 3)]
    f = G.fuse({"operators": ops, "dependencies": deps})
    assert len(f["operators"]) == 5          # fused conv + the four parameter inputs
    epi = G.op_body(_find(f, 1))["epilogue"]
    assert [G.epilogue_name(e) for e in epi] == ["BatchNorm", "ReLU"]
    bn = epi[0]["BatchNorm"]
    assert (bn["gamma_id"], bn["beta_id"], bn["mean_id"], bn["var_id"]) == (10, 11, 12, 13)
    assert set(f["dependencies"]) == {(10, 1), (11, 1), (12, 1), (13, 1)}


def test_residual_fusion():
    ops = [G.conv2d(1, "main_path", 1, 64, 56, 56, 64, 3, 3, 1, 1), G.add(2, "add", 64 * 56 * 56),
           G.relu(3, "relu", 64 * 56 * 56), G.input_op(0, "input")]
    deps = [(0, 1), (0, 2), (1, 2), (2, 3)]
    f = G.fuse({"operators": ops, "dependencies": deps})
    assert len(f["operators"]) == 2
    epi = G.op_body(_find(f, 1))["epilogue"]
    assert [G.epilogue_name(e) for e in epi] == ["ResidualAdd", "ReLU"]
    assert epi[0]["ResidualAdd"]["residual_ptr"] == 0


def test_relu_with_two_consumers_of_the_conv_is_not_fused():
    ops = [G.conv2d(1, "conv", 1, 8, 8, 8, 8, 3, 3, 1, 1), G.relu(2, "relu", 512), G.add(3, "add", 512)]
    f = G.fuse({"operators": ops, "dependencies": [(1, 2), (1, 3), (2, 3)]})
    assert len(f["operators"]) == 3 and G.op_body(_find(f, 1))["epilogue"] == []


def _bottleneck_graph(n=2, cin=64, width=16, h=8):
    return G.bottleneck_graph(n, cin, width, h)


def test_bottleneck_block_fuses_to_three_convs():
    f = G.fuse(_bottleneck_graph())
    kinds = sorted(G.op_kind(o) for o in f["operators"])
    assert kinds.count("Conv2d") == 3 and set(kinds) == {"Conv2d", "Input"}
    assert [G.epilogue_name(e) for e in G.op_body(_find(f, 1))["epilogue"]] == ["BatchNorm", "ReLU"]
    assert [G.epilogue_name(e) for e in G.op_body(_find(f, 4))["epilogue"]] == ["BatchNorm", "ReLU"]
    epi3 = G.op_body(_find(f, 7))["epilogue"]
    assert [G.epilogue_name(e) for e in epi3] == ["BatchNorm", "ResidualAdd", "ReLU"]
    assert epi3[1]["ResidualAdd"]["residual_ptr"] == 0
    assert G.epilogue_string(epi3, False) == "bias+residual+relu"
    # the fused convs chain: x -> c1 -> c2 -> c3, and x also feeds c3 as the residual
    assert {(0, 1), (1, 4), (4, 7), (0, 7)} <= set(f["dependencies"])


def test_json_round_trip_uses_the_serde_layout():
    g = _bottleneck_graph()
    text = G.dump_graph(G.fuse(g))
    parsed = json.loads(text)
    conv = next(o for o in parsed["operators"] if "Conv2d" in o and o["Conv2d"]["op_id"] == 7)
    assert conv["Conv2d"]["epilogue"][2] == "ReLU" and "BatchNorm" in conv["Conv2d"]["epilogue"][0]
    again = G.load_graph(text)
    assert again["operators"] == parsed["operators"]
    with pytest.raises(ValueError, match="Failed to parse JSON"):
        G.load_graph('{"operators": []}')


def test_epilogue_string_rejects_orders_the_kernel_does_not_implement():
    with pytest.raises(ValueError, match="Unsupported epilogue order"):
        G.epilogue_string(["ReLU", {"ResidualAdd": {"residual_ptr": 0}}], False)
    assert G.epilogue_string([], True) == "bias"
    assert G.epilogue_string([], False) == "identity"


def test_batchnorm_folding_matches_conv_then_batchnorm():
    torch.manual_seed(0)
    x = torch.randn(2, 8, 9, 9)
    w = torch.randn(12, 8, 3, 3) * 0.2
    cb = torch.randn(12) * 0.1
    gamma, beta = torch.rand(12) + 0.5, torch.randn(12) * 0.1
    mean, var = torch.randn(12) * 0.2, torch.rand(12) + 0.3
    want = F.batch_norm(F.conv2d(x, w, cb, 1, 1), mean, var, gamma, beta, False, 0.1, 1e-5)
    wf, bf = G.fold_batchnorm(w, gamma, beta, mean, var, 1e-5, cb)
    got = F.conv2d(x, wf, bf, 1, 1)
    assert (got - want).abs().max() < 1e-5 * want.abs().max().clamp(min=1)


@pytest.mark.gpu
def test_fused_bottleneck_graph_runs_on_the_gpu_and_matches_torch():
    torch.manual_seed(1)
    n, cin, width, h = 4, 64, 32, 14
    g = _bottleneck_graph(n, cin, width, h)
    params, names = {}, {G.op_id(o): G.op_body(o)["name"] for o in g["operators"]}
    for oid, name in names.items():
        if name.endswith(".gamma"):
            params[oid] = torch.rand(cin if name.startswith("8.") else width) + 0.5
        elif name.endswith(".var"):
            params[oid] = torch.rand(cin if name.startswith("8.") else width) + 0.3
        elif name.endswith(".beta") or name.endswith(".mean"):
            params[oid] = torch.randn(cin if name.startswith("8.") else width) * 0.2
    params[1] = {"weight": torch.randn(width, cin, 1, 1) * (2.0 / cin) ** 0.5}
    params[4] = {"weight": torch.randn(width, width, 3, 3) * (2.0 / (9 * width)) ** 0.5}
    params[7] = {"weight": torch.randn(cin, width, 1, 1) * (2.0 / width) ** 0.5}
    x = torch.randn(n, cin, h, h).abs()

    def bn(t, conv_id):
        ids = [s for s, d in g["dependencies"] if d == conv_id + 1 and s > 100]
        ga, be, me, va = (params[i] for i in ids)
        return F.batch_norm(t, me, va, ga, be, False, 0.1, 1e-5)

    y1 = F.relu(bn(F.conv2d(x, params[1]["weight"]), 1))
    y2 = F.relu(bn(F.conv2d(y1, params[4]["weight"], None, 1, 1), 4))
    want = F.relu(bn(F.conv2d(y2, params[7]["weight"]), 7) + x)

    runner = G.GraphRunner(G.fuse(g), params, dtype=torch.float32)
    out = runner.run({0: x.cuda()})[7]
    torch.cuda.synchronize()
    err = (out.float().cpu() - want).abs().max() / want.abs().max()
    assert err <= 1.5e-2        # three chained TF32 convs, 5e-3 each
    # the same graph from host memory: input copied in once, only the last conv's output copied back, in image chunks
    host_in = x.contiguous(memory_format=torch.channels_last).pin_memory()
    host_out = torch.empty((n, cin, h, h)).contiguous(memory_format=torch.channels_last).pin_memory()
    for chunks in (1, 3):
        host_out.fill_(float("nan"))
        runner.run_host({0: host_in}, {7: host_out}, chunks=chunks)
        assert torch.equal(host_out, out.cpu()), chunks
