"""The constructor options of the two parallel linears (bias, gather_output, input_is_parallel, sequence_parallel,
keep_master_weight_for_test) and the unpacked-QKV attention block, on gloo ranks against plain full-size math."""
import torch

from dist_utils import run_distributed
from test_modes_cpu import _ref


def _linears(rank, world):
    import torch.distributed as dist
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.parallel.linear import ColumnParallelLinearAG, RowParallelLinearRS, all_gather_seq
    ctx = init_parallel_context("tpsp", device=torch.device("cpu"), backend="library")
    g = ctx.inner_group
    torch.manual_seed(0)                                   # the same full tensors on every rank
    T, din, dmid, dout = 16, 12, 8, 10
    W1, b1 = torch.randn(dmid, din), torch.randn(dmid)
    W2, b2 = torch.randn(dout, dmid), torch.randn(dout)
    x = torch.randn(T, din)
    dy = torch.randn(T, dout)
    t = T // world
    xr = x.clone().requires_grad_(True)
    ref = (xr @ W1.t() + b1) @ W2.t() + b2
    ref.backward(dy)

    def check(col, row, x_in, gather_seq_out):
        col.init_from_master(W1)
        row.init_from_master(W2)
        with torch.no_grad():
            col.bias.copy_(b1[rank * (dmid // world):(rank + 1) * (dmid // world)])
            row.bias.copy_(b2)
        xl = x_in.clone().requires_grad_(True)
        y = row(col(xl))
        if gather_seq_out:                                 # sequence-parallel output: this rank's rows [T/n, out]
            torch.testing.assert_close(all_gather_seq(y.detach(), g), ref.detach(), rtol=1e-5, atol=1e-5)
            (y * dy[rank * t:(rank + 1) * t]).sum().backward()      # each rank owns the loss of its own rows
        else:
            torch.testing.assert_close(y, ref.detach(), rtol=1e-5, atol=1e-5)
            (y * dy).sum().backward()                      # replicated output, replicated loss
        gb2 = row.bias.grad.clone()
        if getattr(row.bias, "grad_sync_group", None) is not None:
            dist.all_reduce(gb2, group=g)
        torch.testing.assert_close(gb2, dy.sum(0), rtol=1e-5, atol=1e-5)
        cols = dmid // world
        torch.testing.assert_close(col.weight.grad, (ref_gW1)[rank * cols:(rank + 1) * cols], rtol=1e-4, atol=1e-5)
        return xl.grad

    # gradient of W1 from the reference graph
    W1r, W2r = W1.clone().requires_grad_(True), W2.clone().requires_grad_(True)
    ((x @ W1r.t() + b1) @ W2r.t() + b2).backward(dy)
    ref_gW1 = W1r.grad

    # (1) sequence parallel, gather_output on the column linear, input_is_parallel=False on the row linear
    col = ColumnParallelLinearAG(din, dmid // world, g, dtype=torch.float32, bias=True, gather_output=True,
                                 keep_master_weight_for_test=True)
    row = RowParallelLinearRS(dmid // world, dout, g, dtype=torch.float32, bias=True, input_is_parallel=False)
    gx = check(col, row, x[rank * t:(rank + 1) * t], True)
    torch.testing.assert_close(gx, xr.grad[rank * t:(rank + 1) * t], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(col.master_weight, W1)
    torch.testing.assert_close(col.get_master_weight(), W1)
    torch.testing.assert_close(row.get_master_weight(), W2)

    # (2) plain tensor parallelism: whole sequence on every rank, all-reduce instead of reduce-scatter
    col = ColumnParallelLinearAG(din, dmid // world, g, dtype=torch.float32, bias=True, sequence_parallel=False)
    row = RowParallelLinearRS(dmid // world, dout, g, dtype=torch.float32, bias=True, sequence_parallel=False)
    gx = check(col, row, x, False)
    torch.testing.assert_close(gx, xr.grad, rtol=1e-4, atol=1e-5)
    return True


def test_parallel_linear_options_world2():
    assert run_distributed(_linears, 2) == {0: True, 1: True}


def _unpacked_qkv(rank, world):
    import torch.distributed as dist
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.models.llama import LlamaForCausalLM
    from odysseus_transformer_b200.parallel.apply import prepare_attn_inputs
    from odysseus_transformer_b200.utils.debug import export_hf_grads
    L = 128
    cfg, sd, batch, ref_loss = _ref("tiny-gqa", L)
    ctx = init_parallel_context("odysseus", device=torch.device("cpu"), backend="library")
    model = LlamaForCausalLM(cfg, "odysseus", ctx, dtype=torch.float32, pack_qkv=False)
    model.init_weights(0)
    assert hasattr(model.layers[0].self_attn, "k_proj") and not hasattr(model.layers[0].self_attn, "qkv_proj")
    pos = torch.arange(L).unsqueeze(0)
    s = prepare_attn_inputs("odysseus", batch[:, :-1], pos, batch[:, 1:], rank, world, "cpu")
    loss = model(s["local_input_ids"], s["local_position_ids"], labels=s["local_target_ids"], global_tokens=L)
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)
    torch.testing.assert_close(total, ref_loss, rtol=1e-4, atol=1e-5)
    grads = export_hf_grads(model)
    for k, v in sd.items():
        torch.testing.assert_close(grads[k], v.grad, rtol=1e-4, atol=2e-6, msg=lambda m: f"unpacked grad {k}: {m}")
    return True


def test_unpacked_qkv_attention_world2():
    assert run_distributed(_unpacked_qkv, 2) == {0: True, 1: True}
