"""The ResNet-50 convolution stack: shape bookkeeping on CPU, per-layer and
end-to-end parity with the oracle on the GPU."""
import pytest
import torch

import oracle
from flagdnn_b200.convstack import ResNet50ConvStack, resnet50_conv_layers, stack_totals


def test_layer_list_matches_published_resnet50_arithmetic():
    layers = resnet50_conv_layers()
    totals = stack_totals(layers, 1024)
    assert totals["convs"] == 53 and totals["unique_shapes"] == 23
    assert totals["flops"] == pytest.approx(8.3705e12, rel=1e-4)       # 8.174 GFLOP per image
    assert totals["bytes"] == pytest.approx(44.65e9, rel=1e-3)
    assert sum(1 for l in layers if not l.relu) == 16 + 4               # third 1x1 of 16 blocks + 4 projections
    assert [l.hw_out for l in layers if l.name.endswith("b0.conv2")] == [56, 28, 14, 7]
    stem = layers[0]
    assert (stem.cin, stem.cout, stem.k, stem.stride, stem.pad, stem.hw_out) == (3, 64, 7, 2, 3, 112)


def _oracle_layer(layer, x, params):
    w, scale, bias = params
    y = oracle.conv2d_torch_cpu(x, w, bias, layer.stride, layer.pad, 1, 1, scale=scale, relu=layer.relu)
    return y.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)


@pytest.mark.gpu
@pytest.mark.parametrize("image,batch", [(224, 2), (64, 5)])
def test_every_layer_matches_oracle_and_chain_matches_end_to_end(native_lib, image, batch):
    import flagdnn_b200 as fd

    stack = ResNet50ConvStack("cuda", seed=7, image=image)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(batch, 3, image, image, generator=g).to(torch.bfloat16)
    x_dev = x.cuda().contiguous(memory_format=torch.channels_last)
    seen = []
    y_dev = stack.forward(x_dev, collect=seen)
    assert len(seen) == 53 and {l.name for l, _, _ in seen} == {l.name for l in stack.layers}
    for layer, inp, out in seen:  # each layer on the very input it consumed
        ref = oracle.conv2d_torch_cpu(inp, stack.params[stack.layers.index(layer)][0],
                                      stack.params[stack.layers.index(layer)][2], layer.stride, layer.pad, 1, 1,
                                      scale=stack.params[stack.layers.index(layer)][1], relu=layer.relu)
        torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-2, atol=1e-2, msg=lambda m: f"{layer.name}: {m}")
    # end to end: the same chain with every convolution done by the CPU oracle (bf16 between layers)
    cpu_params = [tuple(t.cpu() for t in p) for p in stack.params]
    stack_cpu = ResNet50ConvStack.__new__(ResNet50ConvStack)
    stack_cpu.layers, stack_cpu.params = stack.layers, cpu_params
    y_ref = stack_cpu.forward(x.contiguous(memory_format=torch.channels_last), conv=_oracle_layer)
    assert y_dev.shape == y_ref.shape == (batch, 2048, image // 32, image // 32)
    err = (y_dev.float().cpu() - y_ref.float()).abs()
    # 53 layers of bf16 rounding compound; agreement is judged relative to the activation scale
    assert err.max() <= 0.05 * y_ref.float().abs().max() + 0.05
    # shortcut add + ReLU inside each block's last convolution: same chain, one rounding fewer per block
    y_fused = stack.forward(x_dev, fuse_residual=True)
    err = (y_fused.float().cpu() - y_ref.float()).abs()
    assert err.max() <= 0.05 * y_ref.float().abs().max() + 0.05
    assert fd.device_status() == 0


@pytest.mark.gpu
def test_bottleneck_block_graph_replays_as_one_cuda_graph(native_lib):
    """A three-convolution bottleneck (scale + bias folded, ReLU fused) compiled once and replayed."""
    import flagdnn_b200 as fd

    g = torch.Generator().manual_seed(3)

    def t(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).cuda()

    x = t(4, 64, 28, 28).contiguous(memory_format=torch.channels_last)
    w1, w2, w3 = (t(32, 64, 1, 1, std=0.12).contiguous(memory_format=torch.channels_last),
                  t(32, 32, 3, 3, std=0.06).contiguous(memory_format=torch.channels_last),
                  t(64, 32, 1, 1, std=0.17).contiguous(memory_format=torch.channels_last))
    s1, s2, s3 = [(torch.rand(k, generator=g) + 0.5).to(torch.bfloat16).cuda().reshape(1, k, 1, 1) for k in (32, 32, 64)]
    b1, b2, b3 = t(32, std=0.1), t(32, std=0.1), t(64, std=0.1)

    @fd.graph
    def block(x, w1, s1, b1, w2, s2, b2, w3, s3, b3):
        y = fd.relu(fd.bias_add(fd.conv2d(x, w1) * s1, b1))
        y = fd.relu(fd.bias_add(fd.conv2d(y, w2, padding=1) * s2, b2))
        y = fd.bias_add(fd.conv2d(y, w3) * s3, b3)
        return fd.relu(y + x)

    args = [x, w1, s1, b1, w2, s2, b2, w3, s3, b3]
    plain = fd.compile(block, inputs=args, options={"cache": None})
    assert [n.op_type for n in plain.graph.nodes] == ["fused_conv2d_bias_relu", "fused_conv2d_bias_relu",
                                                      "fused_conv2d_bias_add_relu"]
    graphed = fd.compile(block, inputs=args, options={"cache": None, "cuda_graph": True})
    expect = plain.run(*args)
    for _ in range(3):
        got = graphed.run(*args)
    assert torch.equal(got, expect)
    # the same plan with its intermediates in the planned workspace, alone and inside the CUDA graph
    for opts in ({"workspace": True}, {"workspace": True, "cuda_graph": True}):
        planned = fd.compile(block, inputs=args, options={"cache": None, **opts})
        assert planned.plan.workspace_size > 0 and len(planned.plan.memory_plan.blocks) == 2
        for _ in range(2):
            out = planned.run(*args)
        assert torch.equal(out, expect)
        ws = planned._workspaces[x.device]
        assert ws.numel() == planned.plan.workspace_size
    x2 = (x * 0.5).contiguous(memory_format=torch.channels_last)
    assert torch.equal(graphed.run(x2, *args[1:]), plain.run(x2, *args[1:]))

    def cpu_conv(inp, w, s, b, relu, pad=0):
        return oracle.conv2d_torch_cpu(inp, w, b, 1, pad, 1, 1, scale=s.reshape(-1), relu=relu).to(torch.bfloat16)

    y = cpu_conv(x, w1, s1, b1, True)
    y = cpu_conv(y, w2, s2, b2, True, pad=1)
    y = oracle.conv2d_torch_cpu(y, w3, b3, 1, 0, 1, 1, scale=s3.reshape(-1))   # fp32: the fused tail rounds once
    ref = torch.relu(y + x.float().cpu())
    torch.testing.assert_close(expect.float().cpu(), ref, rtol=2e-2, atol=3e-2)


# What the planner chooses for the ResNet-50 layers whose tile counts depend on the batch, at the batches the
# ranks of a strong-scaled run hold (1024 images over 8 and 4 GPUs): (kernel family, tile rows, tile columns,
# pixel group, low-channel mode, grid) on a 148-SM GPU.  A planner change shows up here before it shows up as a
# silent change of tile shape under the parity check below.
RANK_BATCH_PLANS = {
    ("stem", 128): (3, 256, 256, 0, 2, 148),
    ("s2b0.conv2", 128): (3, 256, 256, 2, 0, 148),
    ("s3b0.conv2", 128): (3, 256, 256, 0, 0, 148),
    ("s3b0.conv3", 128): (2, 128, 256, 0, 0, 148),
    ("s3b0.proj", 128): (2, 128, 256, 0, 0, 148),
    ("s3b1.conv1", 128): (3, 256, 256, 0, 0, 148),
    ("s3b1.conv2", 128): (3, 256, 256, 0, 0, 148),
    ("s4b0.conv1", 128): (3, 256, 256, 0, 0, 148),
    ("s4b0.conv2", 128): (3, 256, 256, 0, 0, 100),     # 25 x 2 pair tiles on 74 pairs: long reductions still favour pairs
    ("s4b0.conv3", 128): (2, 128, 256, 0, 0, 148),
    ("s4b0.proj", 128): (3, 256, 256, 0, 0, 148),
    ("s4b1.conv1", 128): (3, 256, 256, 0, 0, 100),
    ("s4b1.conv2", 128): (3, 256, 256, 0, 0, 100),
    ("stem", 256): (3, 256, 256, 0, 2, 148),
    ("s2b0.conv2", 256): (3, 256, 256, 2, 0, 148),
    ("s3b0.conv2", 256): (3, 256, 256, 0, 0, 148),
    ("s3b0.conv3", 256): (2, 128, 256, 0, 0, 148),
    ("s3b0.proj", 256): (2, 128, 256, 0, 0, 148),
    ("s3b1.conv1", 256): (3, 256, 256, 0, 0, 148),
    ("s3b1.conv2", 256): (3, 256, 256, 0, 0, 148),
    ("s4b0.conv1", 256): (3, 256, 256, 0, 0, 148),
    ("s4b0.conv2", 256): (3, 256, 256, 0, 0, 148),
    ("s4b0.conv3", 256): (2, 128, 256, 0, 0, 148),
    ("s4b0.proj", 256): (3, 256, 256, 0, 0, 148),
    ("s4b1.conv1", 256): (3, 256, 256, 0, 0, 148),
    ("s4b1.conv2", 256): (3, 256, 256, 0, 0, 148),
}


def _plan_tuple(fd, x, w, layer):
    p = fd.conv2d_plan(x, w, stride=layer.stride, padding=layer.pad)
    return (p["algo"], p["tile_m"], p["tile_n"], p["pixel_group"], p["low_channel"], p["grid"])


def test_rank_batch_plans_are_the_recorded_ones():
    """CPU side of the table: the planner needs no GPU (148 SMs are assumed when no device is visible)."""
    import flagdnn_b200 as fd

    if torch.cuda.is_available() and torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the table is for a 148-SM GPU")
    by_name = {l.name: l for l in resnet50_conv_layers()}
    for (name, batch), want in RANK_BATCH_PLANS.items():
        l = by_name[name]
        x = torch.empty(batch, l.cin, l.hw_in, l.hw_in, dtype=torch.bfloat16, device="meta", memory_format=torch.channels_last)
        w = torch.empty(l.cout, l.cin, l.k, l.k, dtype=torch.bfloat16, device="meta", memory_format=torch.channels_last)
        assert _plan_tuple(fd, x, w, l) == want, f"{name} at batch {batch}"


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [128, 256])
def test_batch_dependent_layers_at_the_batches_ranks_hold(native_lib, batch):
    """The stem, the stride-2 3x3 layers and every 14x14 / 7x7 layer at 128 and 256 images: the planned tile
    shape is the recorded one, every image agrees with the reference's CPU call in bf16 and sampled images
    (first, last, and two whose rows straddle tile boundaries) with the fp32 oracle."""
    import flagdnn_b200 as fd
    from flagdnn_b200.convstack import make_layer_params, run_layer

    by_name = {l.name: (i, l) for i, l in enumerate(resnet50_conv_layers())}
    g = torch.Generator(device="cuda").manual_seed(batch)
    for (name, b_), want in RANK_BATCH_PLANS.items():
        if b_ != batch:
            continue
        index, l = by_name[name]
        w, scale, bias = make_layer_params(l, index, "cuda")
        x = torch.randn(batch, l.hw_in, l.hw_in, l.cin, generator=g, device="cuda").to(torch.bfloat16).permute(0, 3, 1, 2)
        assert _plan_tuple(fd, x, w, l) == want, f"{name} at batch {batch}"
        y = run_layer(l, x, (w, scale, bias))
        y_cpu = y.float().cpu()
        for i0 in range(0, batch, 64):
            ref16 = oracle.conv2d_torch_cpu(x[i0:i0 + 64], w, bias, l.stride, l.pad, 1, 1, scale=scale, relu=l.relu,
                                            compute_dtype=torch.bfloat16)
            torch.testing.assert_close(y_cpu[i0:i0 + 64], ref16.float(), rtol=1.6e-2, atol=2e-2,
                                       msg=lambda m: f"{name} batch {batch} images {i0}..: {m}")
        picks = [0, batch // 3, batch // 2 + 1, batch - 1]
        ref = oracle.conv2d_torch_cpu(x[picks], w, bias, l.stride, l.pad, 1, 1, scale=scale, relu=l.relu)
        torch.testing.assert_close(y_cpu[picks], ref, rtol=1e-2, atol=1e-2, msg=lambda m: f"{name} batch {batch}: {m}")
    assert fd.device_status() == 0
