"""CPU-only 2-task MPMD pipeline of a 4-layer MLP (fp32, seed 0): layers 0-1 in task A on
virtual device 0, layers 2-3 in task B on device 1, 4 GPipe microbatches, SGD lr 1e-2 for
10 steps. Loss and gradients must match a single-device run to 1e-5."""
import torch

import multimesh_jax_b200 as mm

D_IN = D_H = 512
D_OUT = 10
BATCH = 32
MB = 8
LR = 1e-2


def init_params(seed=0):
    g = torch.Generator().manual_seed(seed)
    dims = [D_IN, D_H, D_H, D_H, D_OUT]
    params = []
    for i in range(4):
        w = torch.randn(dims[i + 1], dims[i], generator=g) / dims[i] ** 0.5
        b = torch.zeros(dims[i + 1])
        params.append((w, b))
    return params


def stage_a(params, x):
    for w, b in params[:2]:
        x = torch.nn.functional.gelu(torch.nn.functional.linear(x, w, b))
    return x


def stage_b(params, h, y):
    (w2, b2), (w3, b3) = params[2], params[3]
    h = torch.nn.functional.gelu(torch.nn.functional.linear(h, w2, b2))
    logits = torch.nn.functional.linear(h, w3, b3)
    return torch.nn.functional.cross_entropy(logits, y, reduction="sum") / BATCH


def make_step(schedule="gpipe"):
    task_a = mm.task(stage_a, name="A", devices=[0])
    task_b = mm.task(stage_b, name="B", devices=[1])

    def loss_fn(params, batch):
        x, y = batch
        return task_b(params, task_a(params, x), y)

    def step(params, batch):
        vg = mm.value_and_grad(loss_fn)
        vg = mm.microbatch(vg, dim=0, size=MB, argnum=1, schedule=schedule)
        loss, grads = vg(params, batch)
        new_params = [(w - LR * gw, b - LR * gb) for (w, b), (gw, gb) in zip(params, grads)]
        return loss, grads, new_params

    return step, loss_fn


def reference_step(params, batch):
    params = [(w.clone().requires_grad_(True), b.clone().requires_grad_(True)) for w, b in params]
    x, y = batch
    loss = stage_b(params, stage_a(params, x), y)
    flat = [t for wb in params for t in wb]
    grads = torch.autograd.grad(loss, flat)
    grads = [(grads[2 * i], grads[2 * i + 1]) for i in range(4)]
    new_params = [(w.detach() - LR * gw, b.detach() - LR * gb) for (w, b), (gw, gb) in zip(params, grads)]
    return loss.detach(), grads, new_params


def _run(schedule):
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    step, _ = make_step(schedule)
    params = init_params(0)
    ref_params = init_params(0)
    x = torch.randn(BATCH, D_IN, generator=g)
    y = torch.randint(0, D_OUT, (BATCH,), generator=g)
    exe = mm.compile_function(step, (params, (x, y)), num_devices=2, backend="cpu")
    names = [t["original_color"] for t in exe.plan["templates"]]
    assert any(n == "A" for n in names) and any(n == "B" for n in names)
    assert any(n == "A_bwd" for n in names) and any(n == "B_bwd" for n in names)
    for it in range(10):
        loss, grads, new_params = exe(params, (x, y))
        ref_loss, ref_grads, ref_new = reference_step(ref_params, (x, y))
        torch.testing.assert_close(loss.full_tensor(), ref_loss, rtol=1e-5, atol=1e-5)
        for (gw, gb), (rw, rb) in zip(grads, ref_grads):
            torch.testing.assert_close(gw.full_tensor(), rw, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(gb.full_tensor(), rb, rtol=1e-5, atol=1e-5)
        params = [(w.full_tensor(), b.full_tensor()) for w, b in new_params]
        ref_params = ref_new
    exe.shutdown()
    return exe


def test_config1_gpipe_matches_single_device():
    exe = _run("gpipe")
    # stage A tasks run on device 0, stage B tasks on device 1
    for t in exe.plan["templates"]:
        if t["original_color"].startswith("A"):
            assert t["device_start"] == 0 and t["num_devices"] == 1
        if t["original_color"].startswith("B"):
            assert t["device_start"] == 1 and t["num_devices"] == 1
    kinds = [op["kind"] for op in exe.plan["ops"]]
    assert kinds.count("reshard") >= 8  # activations forward and gradients backward, per microbatch


def test_config1_1f1b_matches_single_device():
    _run("1f1b")
