"""Host-side logic that needs no GPU: epilogue grammar, shard arithmetic, the ResNet-50 conv table."""
import pytest
import torch

from tracea_b200 import ffi, ops, resnet50, shard


def test_epilogue_grammar_follows_the_reference_runtime_entry():
    # src/interface/python.rs:41-87: '+'-separated, case-insensitive, whitespace-tolerant
    b = torch.zeros(4)
    r = torch.zeros(1, 4, 2, 2)
    assert ops.parse_epilogue(None) == ffi.EPILOGUE_IDENTITY
    assert ops.parse_epilogue("identity") == ffi.EPILOGUE_IDENTITY
    assert ops.parse_epilogue("ReLU") == ffi.EPILOGUE_RELU
    assert ops.parse_epilogue(" bias + relu ", b) == ffi.EPILOGUE_BIAS_RELU
    assert ops.parse_epilogue("bias+silu", b) == ffi.EPILOGUE_BIAS_SILU
    assert ops.parse_epilogue("gelu") == ffi.EPILOGUE_GELU
    assert ops.parse_epilogue("residual+relu", None, r) == ffi.EPILOGUE_RESIDUAL_RELU
    assert ops.parse_epilogue("bias+residual+relu", b, r) == ffi.EPILOGUE_BIAS_RESIDUAL_RELU
    assert ops.parse_epilogue("bias+residual", b, r) == ffi.EPILOGUE_BIAS_RESIDUAL


def test_epilogue_errors_follow_the_reference_runtime_entry():
    with pytest.raises(ValueError, match="no bias argument provided"):
        ops.parse_epilogue("bias+relu")
    with pytest.raises(ValueError, match="no reference provided"):
        ops.parse_epilogue("residual")
    with pytest.raises(ValueError, match="Unknown epilogue op"):
        ops.parse_epilogue("bias+swish", torch.zeros(1))
    with pytest.raises(ValueError, match="Unsupported epilogue sequence"):
        ops.parse_epilogue("relu+bias", torch.zeros(1))


def test_ops_conv2d_shape_checks_match_the_reference_python_op():
    # tracea-python/python/tracea/ops.py:52-61
    with pytest.raises(ValueError, match="Expected NHWC input and KRSC weight"):
        ops.conv2d(torch.zeros(2, 3, 4), torch.zeros(4, 3, 3, 3))
    with pytest.raises(ValueError, match=r"Channel mismatch: x\(8\) vs w\(4\)"):
        ops.conv2d(torch.zeros(1, 5, 5, 8), torch.zeros(16, 3, 3, 4))


@pytest.mark.parametrize("n,world", [(256, 1), (256, 2), (256, 8), (512, 4), (10, 4), (3, 8), (0, 2)])
def test_shards_partition_the_batch(n, world):
    ranges = [shard.shard_range(n, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
        assert a1 == b0 and a0 <= a1
    sizes = shard.shard_sizes(n, world)
    assert sum(sizes) == n and max(sizes) - min(sizes) <= 1


def test_shard_range_rejects_bad_ranks():
    with pytest.raises(ValueError):
        shard.shard_range(8, 2, 2)
    with pytest.raises(ValueError):
        shard.shard_range(8, 0, 0)


def test_resnet50_table():
    specs = resnet50.resnet50_convs()
    assert len(specs) == 53
    assert len({(s.C, s.H, s.K, s.R, s.stride) for s in specs}) == 23
    assert abs(sum(resnet50.conv_flops(s, 1) for s in specs) / 1e9 - 8.174) < 1e-3
    assert abs(sum(resnet50.conv_bytes(s, 512) for s in specs) / 1e9 - 26.9) < 0.05
    # every tensor a conv reads is either a stack input or produced earlier; shapes chain
    produced = {"image": (3, 224), "pooled": (64, 56)}
    for s in specs:
        assert s.src in produced and produced[s.src] == (s.C, s.H), s.name
        ho = resnet50.out_hw(s.H, s.R, s.stride, s.pad)
        if s.res is not None:
            assert produced[s.res] == (s.K, ho), s.name
        produced[s.dst] = (s.K, ho)
    assert produced[specs[-1].dst] == (2048, 7)
    # cross-check against torchvision's architecture when it is importable
    try:
        import torchvision
    except Exception:
        return
    convs = [m for m in torchvision.models.resnet50(weights=None).modules() if isinstance(m, torch.nn.Conv2d)]
    want = sorted((m.in_channels, m.out_channels, m.kernel_size[0], m.stride[0]) for m in convs)
    assert sorted((s.C, s.K, s.R, s.stride) for s in specs) == want


def test_stage3_block_numbers():
    c1, c2, c3 = resnet50.stage3_bottleneck()
    assert (c1.C, c1.K, c1.R) == (1024, 256, 1) and (c2.C, c2.K, c2.R, c2.pad) == (256, 256, 3, 1)
    assert (c3.C, c3.K, c3.res) == (256, 1024, "input")
    assert abs(resnet50.conv_flops(c2, 256) / 1e9 - 59.19) < 0.01
    assert abs(resnet50.conv_bytes(c2, 256) / 1e6 - 52.6) < 0.1
    assert abs(resnet50.conv_bytes(c3, 256) / 1e6 - 231.7) < 0.1


def test_layer_bench_example_parses_its_arguments():
    """examples/layer_bench.py: presets expand to the reference's benchmark layers, dimension counts are checked."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "layer_bench.py")
    spec = importlib.util.spec_from_file_location("layer_bench", path)
    lb = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(lb)
    op, dims, args = lb.parse(["preset", "resnet50-3x3-64"])
    assert (op, dims) == ("conv", [64, 64, 56, 64, 3, 1, 1]) and args.epilogue == "bias+relu"
    op, dims, args = lb.parse(["conv", "256", "64", "56", "64", "3", "1", "1", "--dtype", "f16", "--launch-only"])
    assert dims == [256, 64, 56, 64, 3, 1, 1] and args.dtype == "f16" and args.launch_only
    assert lb.parse(["gemm", "8192", "8192", "8192"])[1] == [8192, 8192, 8192]
    for bad in (["gemm", "1", "2"], ["preset", "nope"], ["conv", "1", "2", "3"]):
        with pytest.raises(SystemExit):
            lb.parse(bad)
