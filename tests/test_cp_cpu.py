"""Ulysses context parallelism on CPU/gloo: a 2-rank CP=2 training step of the tiny Wan DiT
(2 blocks, dim 128, 4 heads x 32, FFN 512, 192 tokens) must reproduce the single-rank step —
loss, reduced gradients and parameters after one AdamW step."""
import pytest
import torch

from dist_utils import run_distributed
from teletron_b200 import ops
from teletron_b200.models import WanModel, wan_config
from teletron_b200.parallel import state as mpu
from teletron_b200.parallel.ddp import DistributedOptimizer, ParamBuffer
from teletron_b200.parallel.ulysses import UlyssesContext


def _problem():
    g = torch.Generator().manual_seed(0)
    x0 = torch.randn(1, 16, 3, 16, 16, generator=g)
    noise = torch.randn(1, 16, 3, 16, 16, generator=g)
    ctx = torch.randn(1, 32, 64, generator=g)
    t = torch.rand(1, generator=g)
    return x0, noise, ctx, t


def _model(cp=None):
    torch.manual_seed(0)
    return WanModel(wan_config("wan-tiny"), cp)


def _step(model, group, grad_scale, local_loss, sharded=False):
    x0, noise, ctx, t = _problem()
    sigma = t
    xt = (1 - sigma) * x0 + sigma * noise
    buf = ParamBuffer(model, shard_world=(2 if sharded else 1))
    opt = DistributedOptimizer(buf, group, lr=1e-4, weight_decay=0.01, clip_grad=0.0, sharded=sharded,
                               grad_scale=grad_scale)
    opt.zero_grad()
    model.return_local_shard = local_loss
    pred = model(xt, t * 1000.0, ctx)
    if local_loss:
        loss = ops.flow_mse(pred, model.local_target_tokens(x0), model.local_target_tokens(noise),
                            scale=1.0 / model.cp.size)
    else:
        loss = ops.flow_mse(pred, x0, noise)
    loss.backward()
    opt.reduce_gradients()
    grads = buf.grads.clone()
    opt.step()
    return loss.detach(), grads, buf.params.clone(), {n: i for n, i in buf.index.items()}


def _worker(rank, world, local_loss, sharded):
    mpu.initialize_model_parallel(context_parallel_size=world)
    cp = UlyssesContext(mpu.get_context_parallel_group(), world, rank)
    model = _model(cp)
    loss, grads, params, _ = _step(model, mpu.get_data_parallel_group(with_context_parallel=True), 1.0,
                                   local_loss, sharded)
    if local_loss:
        torch.distributed.all_reduce(loss)
    return loss, grads, params


@pytest.mark.parametrize("local_loss,sharded", [(True, False), (False, False), (True, True)])
def test_cp2_step_matches_single_rank(local_loss, sharded):
    ref_loss, ref_grads, ref_params, index = _step(_model(), None, 1.0, False)
    outs = run_distributed(_worker, 2, local_loss, sharded)
    for loss, grads, params in outs:
        assert abs(loss.item() - ref_loss.item()) < 1e-5 * max(1.0, abs(ref_loss.item()))
        if not sharded:
            worst = max(((grads[o:o + n] - ref_grads[o:o + n]).norm() / (ref_grads[o:o + n].norm() + 1e-12)).item()
                        for _, (o, n, _) in index.items())
            assert worst < 2e-4, worst
        assert (params - ref_params).abs().max().item() < 2e-6


def _split_gather_worker(rank, world):
    mpu.initialize_model_parallel(context_parallel_size=world)
    cp = UlyssesContext(mpu.get_context_parallel_group(), world, rank)
    x = torch.arange(2 * 98 * 3, dtype=torch.float32).view(2, 98, 3).requires_grad_(True)  # 98 % 4 != 0
    loc = cp.split_tokens(x)
    assert loc.shape[1] == 25
    full = cp.gather_tokens(loc)
    assert torch.equal(full, x.detach())
    (full * (rank + 1)).sum().backward()
    expect = torch.zeros_like(x)
    lo, hi = rank * 25, min((rank + 1) * 25, 98)
    expect[:, lo:hi] = rank + 1
    assert torch.equal(x.grad, expect)
    # attention: 16 heads, sequence not divisible by the group size, against single-device attention
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 98, 16, 8, generator=g) for _ in range(3))
    ref = ops.attention_ref(q, k, v)[0]
    out = cp.attention(cp.split_tokens(q).contiguous(), cp.split_tokens(k).contiguous(),
                       cp.split_tokens(v).contiguous())
    got = cp.gather_tokens(out, 98)
    assert (got - ref).abs().max().item() < 1e-5
    return True


def test_split_gather_and_ulysses_attention_with_padding():
    assert all(run_distributed(_split_gather_worker, 4))


def _heads_not_divisible_worker(rank, world):
    mpu.initialize_model_parallel(context_parallel_size=world)
    cp = UlyssesContext(mpu.get_context_parallel_group(), world, rank)
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(1, 64, 3, 8, generator=g) for _ in range(3))  # 3 heads on 2 ranks
    ref = ops.attention_ref(q, k, v)[0]
    out = cp.attention(*(cp.split_tokens(t).contiguous() for t in (q, k, v)))
    assert (cp.gather_tokens(out, 64) - ref).abs().max().item() < 1e-5
    return True


def test_ulysses_pads_heads():
    assert all(run_distributed(_heads_not_divisible_worker, 2))


def _mixin_names_worker(rank, world):
    import torch

    from teletron_b200.parallel import state as mpu
    from teletron_b200.parallel.ulysses import UlyssesContext

    mpu.initialize_model_parallel(context_parallel_size=world)
    cp = UlyssesContext(mpu.get_context_parallel_group(), world, rank)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 3, 7, 4, generator=g)                 # sequence on dim 2, length 7: padded to 8
    part = cp.split_input(x, dim=2)
    assert part.shape == (2, 3, 4, 4)
    back = cp.gather_output(part, dim=2)
    assert torch.equal(back, x)
    q, k, v = (torch.randn(1, 7, 2 * 8, generator=g) for _ in range(3))
    ql, kl, vl = (cp.split_input(t, dim=1) for t in (q, k, v))
    o = cp.gather_output(cp.forward_attn(ql, kl, vl, num_heads=2), dim=1)
    ref = torch.nn.functional.scaled_dot_product_attention(
        *(t.view(1, 7, 2, 8).transpose(1, 2) for t in (q, k, v))).transpose(1, 2).reshape(1, 7, 16)
    return float((o - ref).abs().max())


def test_reference_mixin_method_names():
    assert max(run_distributed(_mixin_names_worker, 2)) < 1e-5


def _mappings_worker(rank, world):
    import torch
    import torch.distributed as dist

    from teletron_b200.parallel.mappings import (even_sizes, gather_forward_split_backward,
                                                 split_forward_gather_backward)

    assert even_sizes(7, 3) == [3, 2, 2]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 7, 3, generator=g, requires_grad=True)
    # default: 7 over 2 ranks -> 4 + 3; explicit: 2 + 5
    for sizes in (None, [2, 5]):
        part = split_forward_gather_backward(x, None, dim=1, split_sizes=sizes, grad_scale="down")
        want = sizes or [4, 3]
        assert part.shape[1] == want[rank]
        full = gather_forward_split_backward(part, None, dim=1, gather_sizes=want, grad_scale="up")
        assert torch.equal(full, x)
        w = torch.arange(7.0).view(1, 7, 1)
        x.grad = None
        (full * w).sum().backward()
        # gather backward: split, x world ("up"); split backward: gather, / world ("down") -> the plain gradient
        assert torch.allclose(x.grad, w.expand_as(x))
    y = torch.full((3,), float(rank + 1), requires_grad=True)
    z = gather_forward_split_backward(y, None, dim=0)                   # equal sizes, no scaling
    assert z.tolist() == [1.0] * 3 + [2.0] * 3
    z.sum().backward()
    assert y.grad.tolist() == [1.0] * 3
    try:
        split_forward_gather_backward(x, None, dim=1, split_sizes=[1, 1])
    except ValueError:
        return "ok"
    return "no error"


def test_split_gather_mappings_with_uneven_sizes_and_grad_scale():
    assert run_distributed(_mappings_worker, 2) == ["ok", "ok"]


def _cp_sampling_worker(rank, world):
    import torch

    from teletron_b200.infer import WanVideoPipeline
    from teletron_b200.models import WanModel, wan_config
    from teletron_b200.models.encoders import UMT5Encoder, WanVideoVAE
    from teletron_b200.models.encoders.wan_encoder import HashTokenizer
    from teletron_b200.parallel import state as mpu
    from teletron_b200.parallel.ulysses import UlyssesContext

    cp = None
    if world > 1:
        mpu.initialize_model_parallel(context_parallel_size=world)
        cp = UlyssesContext(mpu.get_context_parallel_group(), world, rank)
    torch.manual_seed(0)
    dit = WanModel(wan_config("wan-tiny", text_dim=64), cp).eval()
    t5 = UMT5Encoder(vocab=512, dim=64, dim_attn=64, dim_ffn=128, num_heads=4, num_layers=1)
    pipe = WanVideoPipeline.from_modules(dit, WanVideoVAE(dim=16), t5, None, HashTokenizer(512, 512), device="cpu",
                                         torch_dtype=torch.float32)
    return pipe("a cat", negative_prompt="blurry", height=64, width=48, num_frames=5, num_inference_steps=2, seed=0,
                tiled=False, output_type="latent")


def test_sampling_with_a_context_parallel_dit_matches_one_rank():
    one = run_distributed(_cp_sampling_worker, 1)[0]
    for out in run_distributed(_cp_sampling_worker, 2):
        assert (out - one).abs().max() < 1e-4
