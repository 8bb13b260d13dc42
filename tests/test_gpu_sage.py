"""GPU: the DGL-free GraphSAGE stack (mirror of examples/conv.py, examples/models.py, examples/dataloader.py of the
reference) against a plain-torch restatement on decoded features."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def torch_mean_aggregate(h, indptr, indices):
    n_dst = indptr.numel() - 1
    indices = indices[:int(indptr[-1])]  # the loader's index tensors may carry an unused tail behind indptr[-1]
    deg = indptr[1:] - indptr[:-1]
    dst = torch.repeat_interleave(torch.arange(n_dst, device=h.device), deg)
    out = torch.zeros(n_dst, h.shape[1], device=h.device, dtype=h.dtype).index_add_(0, dst, h[indices])
    return out / deg.clamp_min(1).to(h.dtype)[:, None]


def test_mean_aggregate_forward_and_backward(capi):
    from f2cgt_b200 import sage
    g = torch.Generator(device="cuda").manual_seed(0)
    n_src, n_dst, H = 500, 200, 64
    deg = torch.randint(0, 9, (n_dst,), generator=g, device="cuda")
    indptr = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(deg, 0)])
    indices = torch.randint(0, n_src, (int(indptr[-1]),), generator=g, device="cuda")
    h = torch.randn(n_src, H, generator=g, device="cuda", requires_grad=True)
    w = torch.randn(n_dst, H, generator=g, device="cuda")
    out = sage._MeanAggregate.apply(h, indptr, indices, n_src)
    (out * w).sum().backward()
    got_grad = h.grad.clone()
    h.grad = None
    ref = torch_mean_aggregate(h, indptr, indices)
    (ref * w).sum().backward()
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(got_grad, h.grad, rtol=1e-5, atol=1e-6)


def test_sage_forward_equals_torch_on_decoded_features(capi):
    """Two-level compressed input: the model's output equals the same network evaluated on features decoded row by row."""
    from f2cgt_b200 import ops, sage, synth
    dev = "cuda"
    n, D, hidden, classes = 30000, 128, 64, 10
    indptr, indices = synth.power_law_graph(n, 15, 2.1, seed=1, device=dev)
    g = torch.Generator(device=dev).manual_seed(2)
    vq_codes = torch.randint(0, 256, (n, 4), generator=g, dtype=torch.uint8, device=dev)
    vq_cbs = torch.randn(4, 256, 32, generator=g, device=dev)
    n_hot = 1500
    hot = torch.randperm(n, generator=g, device=dev)[:n_hot]
    slot = torch.full((n,), -1, dtype=torch.int32, device=dev)
    slot[hot] = torch.arange(n_hot, dtype=torch.int32, device=dev)
    sq_codes = torch.randint(-128, 128, (n_hot, D), generator=g, dtype=torch.int8, device=dev)
    sq_cb = synth.sq_codebook_from_sample(torch.randn(5000, D, generator=g, device=dev), D)
    cm = sage.CompressionManager(D, ["sq", "vq"], [(D, 8), (32, 8)], [sq_cb, vq_cbs], [sq_codes, vq_codes], slot)
    full = ops.vq_decompress(vq_codes, vq_cbs, D)
    full[hot] = ops.sq_decompress(sq_codes, sq_cb, 8, D, D)
    torch.manual_seed(0)
    model = sage.SAGE(D, hidden, classes, 3, 0.5, cm).to(dev).eval()
    seeds = torch.randperm(n, generator=g, device=dev)[:128]
    loader = sage.GPUSamplingDataloader(indptr, indices, seeds, 128, (5, 4, 3), shuffle=False)
    input_nodes, output_nodes, blocks = next(iter(loader))
    assert torch.equal(output_nodes, seeds) and torch.equal(blocks[0]["src_nodes"], input_nodes)
    assert torch.equal(cm.decode_rows(input_nodes), full[input_nodes])  # identity-CSC decode is the row decode, bit for bit
    got = model(blocks)
    h = full[input_nodes]
    for i, (layer, b) in enumerate(zip(model.layers, blocks)):
        n_dst = b["dst_nodes"].numel()
        h = layer.fc_self(h[:n_dst]) + layer.fc_neigh(torch_mean_aggregate(h, b["indptr"], b["indices_local"]))
        if i != 2:
            h = torch.relu(h)
    assert got.shape == (128, classes)
    assert torch.allclose(got, h, rtol=1e-4, atol=1e-4)


def test_training_learns_a_feature_rule(capi):
    """Labels that depend on the decoded features of the node itself are learnable through the compressed path."""
    from f2cgt_b200 import ops, sage, synth
    dev = "cuda"
    n, D = 20000, 128
    indptr, indices = synth.power_law_graph(n, 10, 2.1, seed=4, device=dev)
    codes, cb = synth.sq_table_from_normal(n, D, 8, D, seed=5, device=dev)
    cm = sage.CompressionManager(D, ["sq"], [(D, 8)], [cb], [codes])
    feats = ops.sq_decompress(codes, cb, 8, D, D)
    labels = (feats[:, 0] > 0).long() + 2 * (feats[:, 1] > 0).long()
    torch.manual_seed(0)
    model = sage.SAGE(D, 64, 4, 2, 0.0, cm).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    train_ids = torch.arange(8192, device=dev)
    loader = sage.GPUSamplingDataloader(indptr, indices, train_ids, 512, (5, 5), shuffle=True)
    first = last = None
    for epoch in range(6):
        for _, out_nodes, blocks in loader:
            loss = torch.nn.functional.cross_entropy(model(blocks), labels[out_nodes])
            opt.zero_grad()
            loss.backward()
            opt.step()
            first = float(loss.detach()) if first is None else first
            last = float(loss.detach())
    assert last < 0.5 * first, (first, last)


def _two_level_setup(dev="cuda"):
    from f2cgt_b200 import ops, sage, synth
    n, D = 30000, 128
    indptr, indices = synth.power_law_graph(n, 15, 2.1, seed=1, device=dev)
    g = torch.Generator(device=dev).manual_seed(2)
    vq_codes = torch.randint(0, 256, (n, 4), generator=g, dtype=torch.uint8, device=dev)
    vq_cbs = torch.randn(4, 256, 32, generator=g, device=dev)
    n_hot = 1500
    hot = torch.randperm(n, generator=g, device=dev)[:n_hot]
    slot = torch.full((n,), -1, dtype=torch.int32, device=dev)
    slot[hot] = torch.arange(n_hot, dtype=torch.int32, device=dev)
    sq_codes = torch.randint(-128, 128, (n_hot, D), generator=g, dtype=torch.int8, device=dev)
    sq_cb = synth.sq_codebook_from_sample(torch.randn(5000, D, generator=g, device=dev), D)
    cm = sage.CompressionManager(D, ["sq", "vq"], [(D, 8), (32, 8)], [sq_cb, vq_cbs], [sq_codes, vq_codes], slot)
    full = ops.vq_decompress(vq_codes, vq_cbs, D)
    full[hot] = ops.sq_decompress(sq_codes, sq_cb, 8, D, D)
    return n, D, indptr, indices, cm, full, g


def test_sage_gradients_equal_autograd_of_the_plain_network(capi):
    """The hand-written backward of the layers (rows padded to recurring counts and carried through the network) gives
    the gradients autograd computes for the same network written with Linear layers on decoded features."""
    from f2cgt_b200 import sage
    n, D, indptr, indices, cm, full, g = _two_level_setup()
    hidden, classes = 64, 10
    torch.manual_seed(0)
    model = sage.SAGE(D, hidden, classes, 3, 0.0, cm).cuda()
    seeds = torch.randperm(n, generator=g, device="cuda")[:300]  # 300: not a multiple of the row bucket
    loader = sage.GPUSamplingDataloader(indptr, indices, seeds, 300, (5, 4, 3), shuffle=False)
    input_nodes, _, blocks = next(iter(loader))
    y = torch.randint(0, classes, (300,), generator=g, device="cuda")
    got = model(blocks)
    assert got.shape == (300, classes)
    torch.nn.functional.cross_entropy(got, y).backward()
    mine = [p.grad.clone() for p in model.parameters()]
    model.zero_grad(set_to_none=True)
    h = full[input_nodes]
    for i, (layer, b) in enumerate(zip(model.layers, blocks)):
        n_dst = b["dst_nodes"].numel()
        h = layer.fc_self(h[:n_dst]) + layer.fc_neigh(torch_mean_aggregate(h, b["indptr"], b["indices_local"]))
        if i != 2:
            h = torch.relu(h)
    assert torch.allclose(got, h, rtol=1e-4, atol=1e-4)
    torch.nn.functional.cross_entropy(h, y).backward()
    for a, p in zip(mine, model.parameters()):
        assert torch.allclose(a, p.grad, rtol=1e-3, atol=1e-5), float((a - p.grad).abs().max())


def test_hidden_layer_on_unpadded_input(capi):
    """SAGEConv called by hand with exactly n_src rows (fewer than the row bucket of its n_dst): output and gradients."""
    from f2cgt_b200 import sage
    g = torch.Generator(device="cuda").manual_seed(3)
    n_src, n_dst, H = 150, 140, 32
    deg = torch.randint(0, 6, (n_dst,), generator=g, device="cuda")
    indptr = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(deg, 0)])
    indices = torch.randint(0, n_src, (int(indptr[-1]),), generator=g, device="cuda")
    block = dict(dst_nodes=torch.arange(n_dst, device="cuda"), indptr=indptr, indices_local=indices)
    torch.manual_seed(1)
    layer = sage.SAGEConv(H, 16).cuda()
    h = torch.randn(n_src, H, generator=g, device="cuda", requires_grad=True)
    w = torch.randn(n_dst, 16, generator=g, device="cuda")
    out = layer(block, h)
    assert out.shape == (n_dst, 16)
    (out * w).sum().backward()
    got = [h.grad.clone()] + [p.grad.clone() for p in layer.parameters()]
    h.grad = None
    layer.zero_grad(set_to_none=True)
    ref = layer.fc_self(h[:n_dst]) + layer.fc_neigh(torch_mean_aggregate(h, indptr, indices))
    (ref * w).sum().backward()
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
    for a, b in zip(got, [h.grad] + [p.grad for p in layer.parameters()]):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)


def test_loader_builds_the_same_minibatches_ahead_or_in_step(capi):
    """Minibatches built one step early on the side stream (with and without poke() calls in between) are those of the
    in-step loader, tensor for tensor."""
    from f2cgt_b200 import sage, synth
    indptr, indices = synth.power_law_graph(20000, 12, 2.1, seed=7, device="cuda")
    seeds = torch.arange(0, 5000, device="cuda")

    def run(ahead, poke):
        loader = sage.GPUSamplingDataloader(indptr, indices, seeds, 512, (4, 3), shuffle=True, rng_seed=5, ahead=ahead)
        out = []
        for _epoch in range(2):
            for input_nodes, output_nodes, blocks in loader:
                for _ in range(poke):
                    torch.cuda.synchronize()
                    loader.poke()
                out.append([input_nodes.clone(), output_nodes.clone()] +
                           [b[k][:int(b["indptr"][-1])].clone() if k.startswith("indices") else b[k].clone()
                            for b in blocks for k in ("indptr", "indices_global", "indices_local", "src_nodes", "dst_nodes")])
        return out
    base = run(False, 0)
    assert len(base) == 2 * 10
    for ahead, poke in ((True, 0), (True, 1), (True, 3)):
        other = run(ahead, poke)
        assert len(other) == len(base)
        for a, b in zip(base, other):
            assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_direct_fused_adam_equals_torch_adam(capi):
    """The trainer's optimizer calls the fused Adam kernel itself; three steps give torch.optim.Adam(fused=True)'s weights."""
    from f2cgt_b200 import train_graphsage as tg
    if not tg.DirectFusedAdam.available():
        pytest.skip("this torch does not expose the fused Adam kernel")
    torch.manual_seed(0)
    a = [torch.randn(64, 32, device="cuda", requires_grad=True), torch.randn(64, device="cuda", requires_grad=True)]
    b = [t.detach().clone().requires_grad_(True) for t in a]
    mine, ref = tg.DirectFusedAdam(a, lr=0.003), torch.optim.Adam(b, lr=0.003, fused=True)
    for step in range(3):
        g = [torch.randn_like(t) for t in a]
        for t, u, gg in zip(a, b, g):
            t.grad, u.grad = gg.clone(), gg.clone()
        mine.step()
        ref.step()
        mine.lr *= 0.978
        for grp in ref.param_groups:
            grp["lr"] *= 0.978
    for t, u in zip(a, b):
        assert torch.equal(t, u)


def test_bf16_product_operands_stay_close_to_fp32(capi):
    """``sage.products_in(torch.bfloat16)``: same network, product operands rounded to bf16, fp32 everywhere else - output
    and gradients within bf16 rounding of the fp32 run, all finite."""
    from f2cgt_b200 import sage
    n, D, indptr, indices, cm, full, g = _two_level_setup()
    torch.manual_seed(0)
    model = sage.SAGE(D, 64, 10, 3, 0.0, cm).cuda()
    seeds = torch.randperm(n, generator=g, device="cuda")[:256]
    loader = sage.GPUSamplingDataloader(indptr, indices, seeds, 256, (5, 4, 3), shuffle=False)
    _, _, blocks = next(iter(loader))
    y = torch.randint(0, 10, (256,), generator=g, device="cuda")
    want = model(blocks)
    torch.nn.functional.cross_entropy(want, y).backward()
    want_grads = [p.grad.clone() for p in model.parameters()]
    model.zero_grad(set_to_none=True)
    with sage.products_in(torch.bfloat16):
        got = model(blocks)
        torch.nn.functional.cross_entropy(got, y).backward()
    assert got.dtype == torch.float32 and torch.isfinite(got).all()
    # bf16 keeps 8 bits of mantissa: ~0.4 % per operand, through three layers of 64- to 128-term dot products
    scale = float(want.detach().abs().max())
    assert float((got.detach() - want.detach()).abs().max()) < 0.05 * scale
    for a, p in zip(want_grads, model.parameters()):
        assert p.grad.dtype == torch.float32 and torch.isfinite(p.grad).all()
        assert float((p.grad - a).abs().max()) < 0.15 * float(a.abs().max()) + 1e-6
    assert sage._PRODUCT_DTYPE is None  # the context manager restored the default
