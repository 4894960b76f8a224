"""Host-side mirror of the reference interface: argument checks, exception
types and messages (src/flag_dnn/ops/conv2d.py:90-135, 3592-3595), and the
graph API behaviours the reference pins in tests_graph/test_graph.py."""
import pytest
import torch

import flagdnn_b200 as flag_dnn


def test_cpu_tensors_raise_not_implemented(native_lib):
    with pytest.raises(NotImplementedError):
        flag_dnn.conv2d(torch.randn(1, 3, 8, 8), torch.randn(4, 3, 3, 3))
    with pytest.raises(NotImplementedError):
        flag_dnn.fused_conv2d_bias_relu(torch.randn(1, 3, 8, 8), torch.randn(4, 3, 3, 3), torch.randn(4))


@pytest.mark.parametrize("kwargs,exc,msg", [
    (dict(x=torch.randn(3, 8, 8)), RuntimeError, "expects 4D input and weight"),
    (dict(x=torch.zeros(1, 3, 8, 8, dtype=torch.int32), w=torch.zeros(4, 3, 3, 3, dtype=torch.int32)), NotImplementedError, "Unsupported dtype"),
    (dict(w=torch.randn(4, 3, 3, 3).half()), RuntimeError, "same dtype"),
    (dict(b=torch.randn(4).double()), RuntimeError, "bias must have the same dtype"),
    (dict(groups=0), RuntimeError, "groups must be a positive integer"),
    (dict(stride=0), RuntimeError, "stride must be positive"),
    (dict(dilation=(1, 0)), RuntimeError, "dilation must be positive"),
    (dict(padding=-1), RuntimeError, "negative padding"),
    (dict(groups=2), RuntimeError, "divisible by groups"),
    (dict(w=torch.randn(4, 2, 3, 3)), RuntimeError, "input_channels // groups"),
    (dict(b=torch.randn(5)), RuntimeError, "bias shape mismatch"),
    (dict(padding="same", stride=2), RuntimeError, "not supported for strided"),
    (dict(padding="full"), RuntimeError, "padding must be"),
    (dict(stride=(1, 2, 3)), RuntimeError, "expected length 2"),
])
def test_argument_checks_match_reference(kwargs, exc, msg):
    args = dict(x=torch.randn(1, 3, 8, 8), w=torch.randn(4, 3, 3, 3), b=None, stride=1, padding=0, dilation=1, groups=1)
    args.update(kwargs)
    with pytest.raises(exc, match=msg):
        flag_dnn.conv2d(args["x"], args["w"], args["b"], args["stride"], args["padding"], args["dilation"], args["groups"])


def test_conv1d_argument_checks():
    x, w = torch.randn(2, 3, 16), torch.randn(4, 3, 3)
    with pytest.raises(NotImplementedError, match="only supports CUDA"):
        flag_dnn.conv1d(x, w)
    with pytest.raises(RuntimeError, match="2D/3D input and 3D weight"):
        flag_dnn.conv1d(torch.randn(2, 3, 4, 4), w)
    with pytest.raises(RuntimeError, match="length-1 tuple"):
        flag_dnn.conv1d(x, w, stride=(1, 1))


def test_mm_argument_checks():
    with pytest.raises(RuntimeError, match="mat2 must be a matrix"):
        flag_dnn.mm(torch.randn(2, 3), torch.randn(3))
    with pytest.raises(RuntimeError, match=r"cannot be multiplied \(2x3 and 4x5\)"):
        flag_dnn.mm(torch.randn(2, 3), torch.randn(4, 5))
    with pytest.raises(NotImplementedError, match="requires CUDA input"):
        flag_dnn.mm(torch.randn(2, 3), torch.randn(3, 5))


def test_graph_capture_fuses_bias_relu_and_eliminates_dead_node():
    @flag_dnn.graph
    def fn(x, bias):
        y = flag_dnn.bias_add(x, bias)
        out = flag_dnn.relu(y)
        flag_dnn.relu(x)
        return out

    compiled = flag_dnn.compile(fn, inputs=[flag_dnn.TensorSpec("x", (2, 3, 4), "float32"),
                                            flag_dnn.TensorSpec("bias", (3,), "float32")], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_bias_relu"]
    assert compiled.plan.debug_info["fusion"]["bias_activation_fused"] == 1


def test_graph_glue_ops_execute_on_cpu():
    @flag_dnn.graph
    def fn(x, bias):
        return flag_dnn.relu(flag_dnn.bias_add(x, bias))

    x, bias = torch.randn(2, 3, 4), torch.randn(3)
    compiled = flag_dnn.compile(fn, inputs=[x, bias], options={"cache": None})
    torch.testing.assert_close(compiled.run(x, bias), torch.relu(x + bias.reshape(1, 3, 1)))


def test_graph_operator_overload_capture():
    @flag_dnn.graph
    def fn(x, y):
        return flag_dnn.relu(x + y)

    x, y = torch.randn(4, 5), torch.randn(4, 5)
    compiled = flag_dnn.compile(fn, inputs=[x, y], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["add", "relu"]
    torch.testing.assert_close(compiled(x, y), torch.relu(x + y))


def test_graph_conv2d_bias_relu_fuses_in_ir():
    @flag_dnn.graph
    def fn(x, weight, bias):
        y = flag_dnn.conv2d(x, weight, padding=1)
        y = flag_dnn.bias_add(y, bias)
        return flag_dnn.relu(y)

    compiled = flag_dnn.compile(fn, inputs=[flag_dnn.TensorSpec("x", (1, 3, 8, 8), "float32"),
                                            flag_dnn.TensorSpec("weight", (4, 3, 3, 3), "float32"),
                                            flag_dnn.TensorSpec("bias", (4,), "float32")], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_conv2d_bias_relu"]
    node = compiled.graph.nodes[0]
    assert len(node.inputs) == 3 and node.attrs["activation"] == "relu" and node.attrs["padding"] == 1
    assert compiled.plan.debug_info["fusion"]["conv2d_bias_activation_fused"] == 1
    assert compiled.plan.debug_info["kernel_candidates"][0]["op_type"] == "fused_conv2d_bias_relu"
    assert compiled.plan.output_specs[0].shape == (1, 4, 8, 8)


def test_graph_conv_bias_without_relu_folds_bias():
    @flag_dnn.graph
    def fn(x, weight, bias):
        return flag_dnn.bias_add(flag_dnn.conv2d(x, weight, stride=2), bias)

    compiled = flag_dnn.compile(fn, inputs=[flag_dnn.TensorSpec("x", (1, 3, 9, 9), "float16"),
                                            flag_dnn.TensorSpec("weight", (4, 3, 3, 3), "float16"),
                                            flag_dnn.TensorSpec("bias", (4,), "float16")], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d"]
    assert len(compiled.graph.nodes[0].inputs) == 3
    assert compiled.plan.debug_info["fusion"]["conv2d_bias_folded"] == 1
    assert compiled.plan.output_specs[0].shape == (1, 4, 4, 4)


def test_graph_fusion_needs_single_user_and_unbiased_conv():
    @flag_dnn.graph
    def two_users(x, weight, bias):
        y = flag_dnn.conv2d(x, weight)
        return flag_dnn.relu(flag_dnn.bias_add(y, bias)), y

    specs = [flag_dnn.TensorSpec("x", (1, 3, 8, 8), "float32"), flag_dnn.TensorSpec("w", (4, 3, 3, 3), "float32"),
             flag_dnn.TensorSpec("b", (4,), "float32")]
    compiled = flag_dnn.compile(two_users, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d", "fused_bias_relu"]

    @flag_dnn.graph
    def biased(x, weight, bias):
        return flag_dnn.relu(flag_dnn.bias_add(flag_dnn.conv2d(x, weight, bias), bias))

    compiled = flag_dnn.compile(biased, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d", "fused_bias_relu"]


def test_graph_fusion_can_be_disabled(monkeypatch):
    @flag_dnn.graph
    def fn(x, weight, bias):
        return flag_dnn.relu(flag_dnn.bias_add(flag_dnn.conv2d(x, weight), bias))

    specs = [flag_dnn.TensorSpec("x", (1, 3, 8, 8), "float32"), flag_dnn.TensorSpec("w", (4, 3, 3, 3), "float32"),
             flag_dnn.TensorSpec("b", (4,), "float32")]
    compiled = flag_dnn.compile(fn, inputs=specs, options={"cache": None, "fusion": False})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d", "bias_add", "relu"]
    monkeypatch.setenv("FLAGDNN_GRAPH_FUSION", "0")
    compiled = flag_dnn.compile(fn, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d", "bias_add", "relu"]


def test_graph_scale_pattern_folds_with_and_without_relu():
    specs = [flag_dnn.TensorSpec("x", (1, 8, 8, 8), "bfloat16"), flag_dnn.TensorSpec("w", (16, 8, 1, 1), "bfloat16"),
             flag_dnn.TensorSpec("s", (16, 1, 1), "bfloat16"), flag_dnn.TensorSpec("b", (16,), "bfloat16")]

    @flag_dnn.graph
    def no_relu(x, w, s, b):
        return flag_dnn.bias_add(flag_dnn.conv2d(x, w) * s, b)

    compiled = flag_dnn.compile(no_relu, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d"]
    assert len(compiled.graph.nodes[0].inputs) == 4
    assert compiled.plan.debug_info["fusion"]["conv2d_scale_bias_folded"] == 1

    @flag_dnn.graph
    def spatial_scale(x, w, s, b):  # not a per-channel vector: must not be absorbed
        return flag_dnn.relu(flag_dnn.bias_add(flag_dnn.conv2d(x, w) * s, b))

    specs[2] = flag_dnn.TensorSpec("s", (1, 1, 8, 8), "bfloat16")
    compiled = flag_dnn.compile(spatial_scale, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d", "mul", "fused_bias_relu"]

    # a plain (K,) vector multiplies along W (torch broadcasting), which is only expressible when W == K:
    # it is not a per-channel scale and must stay a separate node
    specs_wk = [flag_dnn.TensorSpec("x", (1, 8, 4, 16), "bfloat16"), flag_dnn.TensorSpec("w", (16, 8, 1, 1), "bfloat16"),
                flag_dnn.TensorSpec("s", (16,), "bfloat16"), flag_dnn.TensorSpec("b", (16,), "bfloat16")]
    for fn in (no_relu, spatial_scale):
        compiled = flag_dnn.compile(fn, inputs=specs_wk, options={"cache": None})
        kinds = [n.op_type for n in compiled.graph.nodes]
        assert "mul" in kinds and all(len(n.inputs) <= 3 for n in compiled.graph.nodes if n.op_type == "conv2d")
        assert "conv2d_scale_bias_folded" not in compiled.plan.debug_info["fusion"]
    # ... except for a single output channel, where the one-element vector is the channel's scale
    specs_k1 = [flag_dnn.TensorSpec("x", (1, 8, 4, 4), "bfloat16"), flag_dnn.TensorSpec("w", (1, 8, 1, 1), "bfloat16"),
                flag_dnn.TensorSpec("s", (1,), "bfloat16"), flag_dnn.TensorSpec("b", (1,), "bfloat16")]
    compiled = flag_dnn.compile(no_relu, inputs=specs_k1, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d"] and len(compiled.graph.nodes[0].inputs) == 4


def test_graph_residual_tail_becomes_one_node():
    specs = [flag_dnn.TensorSpec("x", (2, 8, 8, 8), "bfloat16"), flag_dnn.TensorSpec("w", (8, 8, 1, 1), "bfloat16"),
             flag_dnn.TensorSpec("s", (8, 1, 1), "bfloat16"), flag_dnn.TensorSpec("b", (8,), "bfloat16"),
             flag_dnn.TensorSpec("wp", (8, 8, 1, 1), "bfloat16")]

    @flag_dnn.graph
    def identity_block(x, w, s, b, wp):
        return flag_dnn.relu(x + flag_dnn.bias_add(flag_dnn.conv2d(x, w) * s, b))    # conv on the right of the add

    compiled = flag_dnn.compile(identity_block, inputs=specs, options={"cache": None})
    nodes = compiled.graph.nodes
    assert [n.op_type for n in nodes] == ["fused_conv2d_bias_add_relu"]
    g = compiled.graph
    assert nodes[0].inputs[:3] == [g.inputs[0], g.inputs[1], g.inputs[0]]            # x, w, shortcut = x
    assert nodes[0].inputs[3:] == [g.inputs[3], g.inputs[2]]                         # bias, scale
    assert compiled.plan.debug_info["fusion"]["conv2d_residual_activation_fused"] == 1

    @flag_dnn.graph
    def projection_block(x, w, s, b, wp):
        main = flag_dnn.bias_add(flag_dnn.conv2d(x, w) * s, b)
        return flag_dnn.relu(main + flag_dnn.conv2d(x, wp))     # shortcut produced after the main convolution

    compiled = flag_dnn.compile(projection_block, inputs=specs, options={"cache": None})
    kinds = [n.op_type for n in compiled.graph.topological_nodes()]
    assert sorted(kinds) == ["conv2d", "fused_conv2d_bias_add_relu"] and kinds[-1] == "fused_conv2d_bias_add_relu"
    compiled.graph.lint()

    @flag_dnn.graph
    def broadcast_add(x, w, s, b, wp):
        return flag_dnn.relu(flag_dnn.conv2d(x, w) + s)          # not a same-shape shortcut: stays unfused

    compiled = flag_dnn.compile(broadcast_add, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d", "add", "relu"]

    @flag_dnn.graph
    def shared_conv(x, w, s, b, wp):
        y = flag_dnn.conv2d(x, w)
        return flag_dnn.relu(y + x), y                           # the convolution has a second user

    compiled = flag_dnn.compile(shared_conv, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["conv2d", "add", "relu"]


def test_graph_gelu_patterns():
    specs = [flag_dnn.TensorSpec("x", (1, 8, 8, 8), "float16"), flag_dnn.TensorSpec("w", (16, 8, 3, 3), "float16"),
             flag_dnn.TensorSpec("b", (16,), "float16")]

    @flag_dnn.graph
    def conv_gelu(x, w, b):
        return flag_dnn.gelu(flag_dnn.bias_add(flag_dnn.conv2d(x, w, padding=1), b), approximate="tanh")

    compiled = flag_dnn.compile(conv_gelu, inputs=specs, options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_conv2d_bias_gelu"]
    assert compiled.graph.nodes[0].attrs["approximate"] == "tanh" and compiled.graph.nodes[0].attrs["activation"] == "gelu"

    @flag_dnn.graph
    def bias_gelu(x, w, b):                       # no convolution upstream: the reference's fused_bias_gelu
        return flag_dnn.gelu(flag_dnn.bias_add(x, w))

    compiled = flag_dnn.compile(bias_gelu, inputs=[specs[0], flag_dnn.TensorSpec("b8", (8,), "float16"), specs[2]],
                                options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_bias_gelu"]
    x = torch.randn(1, 8, 8, 8, dtype=torch.float32)
    b8 = torch.randn(8, dtype=torch.float32)
    compiled32 = flag_dnn.compile(bias_gelu, inputs=[x, b8, b8], options={"cache": None})
    torch.testing.assert_close(compiled32.run(x, b8, b8), torch.nn.functional.gelu(x + b8.view(1, 8, 1, 1)))


def test_pooling_ops_capture_and_refuse_cpu_eagerly():
    @flag_dnn.graph
    def tail(x):
        return flag_dnn.adaptive_avg_pool2d(flag_dnn.max_pool2d(x, 3, stride=2, padding=1, ceil_mode=True), (1, None))

    compiled = flag_dnn.compile(tail, inputs=[flag_dnn.TensorSpec("x", (2, 8, 15, 15), "float32")], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["max_pool2d", "adaptive_avg_pool2d"]
    x = torch.randn(2, 8, 15, 15)
    ref = torch.nn.functional.adaptive_avg_pool2d(torch.nn.functional.max_pool2d(x, 3, 2, 1, ceil_mode=True), (1, None))
    out = compiled.run(x)                        # CPU tensors: shape-checking glue, as for the other glue ops
    assert out.shape == (2, 8, 1, 8) and torch.allclose(out, ref)
    with pytest.raises(NotImplementedError, match="requires CUDA input"):
        flag_dnn.max_pool2d(x, 2)
    with pytest.raises(NotImplementedError, match="requires CUDA input"):
        flag_dnn.adaptive_avg_pool2d(x, 1)


def test_memory_plan_places_intermediates_and_reuses_dead_blocks():
    """Lifetimes and first-fit reuse as the reference plans them (src/flag_dnn/graph/memory.py:125-199)."""
    specs = [flag_dnn.TensorSpec("x", (2, 8, 16, 16), "float32"), flag_dnn.TensorSpec("w", (8, 8, 3, 3), "float32"),
             flag_dnn.TensorSpec("b", (8,), "float32")]

    @flag_dnn.graph
    def chain(x, w, b):
        a = flag_dnn.conv2d(x, w, padding=1)          # value A: dies after the second convolution
        c = flag_dnn.conv2d(a, w, padding=1)          # value C
        d = flag_dnn.conv2d(c, w, padding=1)          # value D: can take A's block
        return flag_dnn.relu(flag_dnn.bias_add(flag_dnn.conv2d(d, w, padding=1), b))

    compiled = flag_dnn.compile(chain, inputs=specs, options={"cache": None})
    plan = compiled.plan.memory_plan
    nbytes = 2 * 8 * 16 * 16 * 4
    assert len(plan.lifetimes) == 3 and all(t.size_bytes == nbytes for t in plan.lifetimes)
    births = sorted((t.birth, t.last_use) for t in plan.lifetimes)
    assert births == [(0, 1), (1, 2), (2, 3)]
    assert len(plan.blocks) == 2 and plan.workspace_size == 2 * nbytes        # two live at a time, the third reuses
    offsets = [plan.allocations[t.value_id].offset for t in sorted(plan.lifetimes, key=lambda t: t.birth)]
    assert offsets[0] == offsets[2] != offsets[1] and all(o % 256 == 0 for o in offsets)
    d = compiled.plan.debug_info["memory"]
    assert set(d) >= {"workspace_size", "lifetimes", "reusable_value_ids", "blocks", "allocations"}
    assert compiled.plan.workspace_size == plan.workspace_size
    # graph outputs and inputs are never placed
    planned = set(plan.allocations)
    assert not planned & set(compiled.graph.inputs) and not planned & set(compiled.graph.outputs)


def test_graph_memory_plan_cache_hit():
    cache = flag_dnn.PlanCache(enable_disk=False)

    @flag_dnn.graph
    def fn(x, bias):
        return flag_dnn.relu(flag_dnn.bias_add(x, bias))

    specs = [flag_dnn.TensorSpec("x", (2, 3), "float32"), flag_dnn.TensorSpec("bias", (3,), "float32")]
    first = flag_dnn.compile(fn, inputs=specs, options={"cache": cache})
    second = flag_dnn.compile(fn, inputs=specs, options={"cache": cache})
    assert first.plan.workspace_size >= 0 and first.plan.memory_plan is not None
    assert second.plan.debug_info["cache_hit"] is True
    assert second.plan.debug_info["cache_layer"] == "memory"


def test_graph_autotune_option_is_recorded():
    @flag_dnn.graph
    def fn(x, bias):
        return flag_dnn.relu(flag_dnn.bias_add(x, bias))

    compiled = flag_dnn.compile(fn, inputs=[torch.randn(2, 3), torch.randn(3)],
                                options={"cache": None, "autotune": True, "autotune_repeat": 1})
    assert compiled.plan.debug_info["autotune"]["enabled"] is True
    assert compiled.plan.debug_info["candidate_count"] >= 1


def test_graph_ops_namespace_capture_keeps_attrs():
    @flag_dnn.graph
    def fn(x, y):
        return flag_dnn.ops.add(x, y, compute_data_type="float32", name="add")

    x, y = torch.randn(4, 5), torch.randn(4, 5)
    compiled = flag_dnn.compile(fn, inputs=[x, y], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["add"]
    assert compiled.graph.nodes[0].attrs["name"] == "add"
    torch.testing.assert_close(compiled(x, y), x + y)


def test_executor_validates_inputs_and_refuses_cpu_convolution():
    @flag_dnn.graph
    def fn(x, weight, bias):
        return flag_dnn.relu(flag_dnn.bias_add(flag_dnn.conv2d(x, weight), bias))

    x, w, b = torch.randn(1, 3, 8, 8), torch.randn(4, 3, 3, 3), torch.randn(4)
    compiled = flag_dnn.compile(fn, inputs=[x, w, b], options={"cache": None})
    with pytest.raises(RuntimeError, match="shape"):
        compiled.run(torch.randn(2, 3, 8, 8), w, b)
    with pytest.raises(RuntimeError, match="dtype"):
        compiled.run(x.double(), w, b)
    with pytest.raises(RuntimeError, match="stride"):
        compiled.run(x.contiguous(memory_format=torch.channels_last), w, b)
    with pytest.raises(RuntimeError, match="expects 3 inputs"):
        compiled.run(x, w)
    with pytest.raises(NotImplementedError, match="CUDA tensors only"):
        compiled.run(x, w, b)  # no CPU implementation of the hot path in this package


def test_conv2d_plan_reports_library_decision(native_lib):
    x = torch.empty(256, 256, 14, 14, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = torch.empty(256, 256, 3, 3, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    plan = flag_dnn.conv2d_plan(x, w, padding=1)
    assert plan["algo"] == 3 and plan["tile_n"] == 256 and plan["x_repacked"] == 0 and plan["w_packed"] == 0


def test_tune_tool_needs_a_gpu_and_says_so():
    """`python -m flagdnn_b200.tune` measures on the device: without one it explains itself and exits with 2
    instead of falling back to anything."""
    import subprocess
    import sys

    from conftest import ROOT

    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the tool would run its sweep")
    proc = subprocess.run([sys.executable, "-m", "flagdnn_b200.tune", "--batch", "2"], capture_output=True, text=True,
                          cwd=ROOT, timeout=300)
    assert proc.returncode == 2
    assert "needs a CUDA device" in proc.stderr
