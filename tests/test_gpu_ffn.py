"""(c) Grouped expert FFN on capacity-strided rows against the oracle's ``expert_ffn``
(forward, and backward through autograd).  fp32 runs on the CUDA-core kernels (rtol 1e-5),
bf16 on the tcgen05 kernels (rtol 1e-2) and, to bisect, on the CUDA-core kernels too."""
import pytest
import torch

from oracle import moe_ref as O
from util import assert_close, rel_fro

pytestmark = pytest.mark.gpu


class Case:
    def __init__(self, M, F, L, n_src, Cs, counts, dtype, seed=0, bias=True, act="gelu",
                 gelu_bwd="exact"):
        g = torch.Generator().manual_seed(seed)
        self.M, self.F, self.L, self.n_src, self.Cs, self.dtype, self.act = M, F, L, n_src, Cs, dtype, act
        self.gelu_bwd = gelu_bwd
        self.counts = torch.tensor(counts, dtype=torch.int32).view(n_src, L)
        self.w1 = (torch.randn(L, F, M, generator=g) * 0.05).to(dtype)
        self.w2 = (torch.randn(L, F, M, generator=g) * 0.05).to(dtype)
        self.b1 = (torch.randn(L, F, generator=g) * (0.1 if bias else 0)).to(dtype)
        self.b2 = (torch.randn(L, M, generator=g) * (0.1 if bias else 0)).to(dtype)
        rows = n_src * L * Cs
        # valid rows random, pad rows of each 128-row tile zero, everything beyond NaN
        self.x = torch.full((n_src, L, Cs, M), float("nan")).to(dtype)
        self.dout = torch.full((n_src, L, Cs, M), float("nan")).to(dtype)
        for w in range(n_src):
            for l in range(L):
                c = int(self.counts[w, l])
                pad = (c + 127) // 128 * 128
                self.x[w, l, :pad] = 0
                self.dout[w, l, :pad] = 0
                self.x[w, l, :c] = torch.randn(c, M, generator=g).to(dtype)
                self.dout[w, l, :c] = torch.randn(c, M, generator=g).to(dtype)

    def expert_rows(self, t, l):
        return torch.cat([t[w, l, :int(self.counts[w, l])] for w in range(self.n_src)], 0)

    def oracle(self, l):
        """Forward and backward of local expert l on its valid rows: fp32 arithmetic, stored
        tensors rounded to the case's dtype (identity for fp32)."""
        x = self.expert_rows(self.x, l).float()
        dout = self.expert_rows(self.dout, l).float()
        r = O.ffn_explicit(x, self.w1[l].float(), self.b1[l].float(), self.w2[l].float(),
                           self.b2[l].float(), dout, self.dtype, act=self.act, gelu_bwd=self.gelu_bwd)
        return r["out"], r["dx"], [r["gw1"], r["gb1"], r["gw2"], r["gb2"]]


def run_gpu(case, e_begin=0, e_end=None, backend=0, accumulate=False, slots=None, grads=None,
            compact=0):
    from mole_b200 import ops
    c = case
    e_end = c.L if e_end is None else e_end
    dev = torch.device("cuda")
    n_slots = c.L if slots is None else max(slots) + 1
    desc = ops.make_ffn_desc(c.dtype, c.act, c.gelu_bwd, c.M, c.F, c.L, c.n_src, c.Cs, e_begin, e_end,
                             n_slots, accumulate, backend, compact=compact)
    ws = ops.ffn_workspace(desc, dev)
    rows = c.n_src * c.L * c.Cs
    x = c.x.view(rows, c.M).cuda()
    dout = c.dout.view(rows, c.M).cuda()
    w1, b1, w2, b2 = (t.cuda() for t in (c.w1, c.b1, c.w2, c.b2))
    if slots is not None:      # scatter the weights into their slots
        def place(t):
            o = torch.zeros(n_slots, *t.shape[1:], dtype=t.dtype, device=dev)
            for l, s in enumerate(slots):
                o[s] = t[l]
            return o
        w1, b1, w2, b2 = (place(t) for t in (w1, b1, w2, b2))
    nan = float("nan")
    x1 = torch.full((rows, c.F), nan, dtype=c.dtype, device=dev)
    h = torch.full((rows, c.F), nan, dtype=c.dtype, device=dev)
    out = torch.full((rows, c.M), nan, dtype=c.dtype, device=dev)
    counts = c.counts.flatten().cuda()
    ops.ffn_fwd(desc, counts, x, w1, b1, w2, b2, x1, h, out, ws, slots)
    dx1 = torch.full((rows, c.F), nan, dtype=c.dtype, device=dev)
    dx = torch.full((rows, c.M), nan, dtype=c.dtype, device=dev)
    if grads is None:
        grads = [torch.full_like(t, nan) for t in (w1, b1, w2, b2)]
    ops.ffn_bwd(desc, counts, dout, x, x1, h, w1, w2, dx1, dx, grads[0], grads[1], grads[2],
                grads[3], ws, slots, slots)
    assert ops.device_fault() == 0
    torch.cuda.synchronize()
    shape = (c.n_src, c.L, c.Cs)
    return out.view(*shape, c.M).cpu(), dx.view(*shape, c.M).cpu(), [g.cpu() for g in grads]


def check(case, out, dx, grads, experts, slots=None, wscale=1.0):
    names = ("gW1", "gb1", "gW2", "gb2")
    for l in experts:
        o_ref, dx_ref, g_ref = case.oracle(l)
        n = o_ref.shape[0]
        s = l if slots is None else slots[l]
        if n:
            assert_close(case.expert_rows(out, l), o_ref, case.dtype, f"out, expert {l}")
            assert_close(case.expert_rows(dx, l), dx_ref, case.dtype, f"dx, expert {l}")
        for name, got, ref in zip(names, grads, g_ref):
            if n == 0:
                assert (got[s] == 0).all(), f"{name}, empty expert {l}: gradient must be zero"
            else:
                assert_close(got[s], ref, case.dtype, f"{name}, expert {l}", scale=wscale)


RAGGED = [0, 1, 127, 128, 129, 200, 256, 5]


def test_ffn_fp32_cuda_cores():
    case = Case(M=128, F=256, L=8, n_src=1, Cs=256, counts=RAGGED, dtype=torch.float32)
    out, dx, grads = run_gpu(case)
    check(case, out, dx, grads, range(8), wscale=4.0)


def test_ffn_fp32_two_sources_and_relu():
    counts = [3, 130, 0, 64, 128, 0, 0, 17]        # [n_src=2][L=4]; expert 2 is empty everywhere
    case = Case(M=64, F=192, L=4, n_src=2, Cs=256, counts=counts, dtype=torch.float32, act="relu")
    out, dx, grads = run_gpu(case)
    check(case, out, dx, grads, range(4), wscale=4.0)


@pytest.mark.parametrize("backend", [1, 2, 3, 4],
                         ids=["cuda_cores", "tcgen05_one_cta", "tcgen05_cta_pair", "tcgen05_panel"])
def test_ffn_bf16(backend):
    case = Case(M=256, F=512, L=8, n_src=1, Cs=256, counts=RAGGED, dtype=torch.bfloat16, seed=1)
    out, dx, grads = run_gpu(case, backend=backend)
    check(case, out, dx, grads, range(8))


def test_ffn_bf16_tcgen05_narrow_tiles_two_sources():
    # M = 128 exercises the 128-column tile variant; two source ranks per expert
    counts = [100, 0, 256, 1, 0, 0, 130, 128]
    case = Case(M=128, F=384, L=4, n_src=2, Cs=256, counts=counts, dtype=torch.bfloat16, seed=2)
    out, dx, grads = run_gpu(case)
    check(case, out, dx, grads, range(4))


@pytest.mark.parametrize("backend", [2, 3, 4])
def test_ffn_bf16_four_sources_packed_per_expert(backend):
    """Four source ranks per expert: the tensor-core path packs each expert's rows of all sources
    into one run (rows cross 128-row tile edges inside a source's chunk), computes there and
    scatters out / dx back to the (source, expert) chunks.  Checked against the oracle, and
    against the same call with packing switched off, on a sub-range of experts."""
    counts = [100, 0, 256, 1, 7, 128,
              30, 0, 129, 0, 250, 128,
              0, 0, 5, 200, 255, 128,
              127, 0, 1, 56, 3, 128]            # [n_src=4][L=6]; expert 1 is empty everywhere
    case = Case(M=256, F=512, L=6, n_src=4, Cs=256, counts=counts, dtype=torch.bfloat16, seed=7)
    out, dx, grads = run_gpu(case, backend=backend)
    check(case, out, dx, grads, range(6))
    out_r, dx_r, grads_r = run_gpu(case, e_begin=2, e_end=5, backend=backend)
    out_c, dx_c, grads_c = run_gpu(case, e_begin=2, e_end=5, backend=backend, compact=2)
    check(case, out_r, dx_r, grads_r, (2, 3, 4))
    for l in (2, 3, 4):
        assert_close(case.expert_rows(out_r, l), case.expert_rows(out_c, l), case.dtype, f"out {l}")
        assert_close(case.expert_rows(dx_r, l), case.expert_rows(dx_c, l), case.dtype, f"dx {l}")
    for l in (0, 1, 5):
        assert torch.isnan(out_r[:, l].float()).all()


@pytest.mark.parametrize("backend", [0, 3, 4], ids=["default", "tcgen05_cta_pair", "tcgen05_panel"])
def test_ffn_bf16_expert_range_slots_and_accumulate(backend):
    """A record of experts [2, 5) with weights living in permuted slots and gradients
    accumulated onto existing values (the offload pipeline's way of calling the FFN)."""
    from mole_b200 import ops
    case = Case(M=256, F=256, L=6, n_src=1, Cs=128, counts=[5, 9, 100, 128, 64, 3],
                dtype=torch.bfloat16, seed=3)
    slots = [7, 6, 3, 0, 5, 1]
    base = [torch.full((8, 256, 256), 0.5), torch.full((8, 256), 0.5),
            torch.full((8, 256, 256), 0.5), torch.full((8, 256), 0.5)]
    grads = [b.bfloat16().cuda() for b in base]
    out, dx, grads = run_gpu(case, e_begin=2, e_end=5, accumulate=True, slots=slots, grads=grads,
                             backend=backend)
    for l in (2, 3, 4):
        o_ref, dx_ref, g_ref = case.oracle(l)
        assert_close(case.expert_rows(out, l), o_ref, case.dtype, f"out {l}")
        assert_close(case.expert_rows(dx, l), dx_ref, case.dtype, f"dx {l}")
        for got, ref in zip(grads, g_ref):
            assert_close(got[slots[l]], ref + 0.5, case.dtype, f"accumulated grad {l}")
    for l in (0, 1, 5):        # untouched experts: outputs never written, gradients unchanged
        assert torch.isnan(out[0, l].float()).all()
        for got in grads:
            assert (got[slots[l]] == 0.5).all()


def test_ffn_bf16_full_size_spot_check():
    """Benchmark shape (64 experts, M = 1024, F = 4096, ~512 rows per expert): the tcgen05 path
    against the oracle on a sample of rows, and against the CUDA-core path through the Frobenius
    norm of every output."""
    g = torch.Generator().manual_seed(5)
    L, M, F, Cs = 64, 1024, 4096, 640
    counts = torch.randint(400, 641, (L,), generator=g).tolist()
    counts[3], counts[10] = 0, 640
    case = Case(M, F, L, 1, Cs, counts, torch.bfloat16, seed=6)
    out, dx, grads = run_gpu(case)
    out2, dx2, grads2 = run_gpu(case, backend=1)
    out3, dx3, grads3 = run_gpu(case, backend=2)
    out, dx, grads = run_gpu(case, backend=3)
    valid = torch.zeros(1, L, Cs, dtype=torch.bool)
    for l in range(L):
        valid[0, l, :counts[l]] = True
    assert rel_fro(out[valid], out2[valid]) < 4e-3
    assert rel_fro(dx[valid], dx2[valid]) < 4e-3
    for a, b in zip(grads, grads2):
        assert rel_fro(a, b) < 4e-3
    # the CTA-pair kernel and the one-CTA kernel accumulate in the same order: identical bits
    assert torch.equal(out[valid], out3[valid]) and torch.equal(dx[valid], dx3[valid])
    for i, (a, b) in enumerate(zip(grads, grads3)):
        if i == 1:      # FC1 bias gradient: summed in the CTA-pair kernel's dX2 epilogue, in another order
            assert rel_fro(a, b) < 2e-3
        else:
            assert torch.equal(a, b)
    # the panel kernel (two or three row panels per expert here) sums over K in the same order
    out4, dx4, grads4 = run_gpu(case, backend=4)
    assert torch.equal(out[valid], out4[valid]) and torch.equal(dx[valid], dx4[valid])
    for i, (a, b) in enumerate(zip(grads, grads4)):
        if i == 1:
            # the FC1 bias gradient comes out of the panel kernel's dX2 epilogue: the same bf16
            # values of dX1 added in another (fixed) order, so a last-bit difference may remain
            assert rel_fro(a, b) < 2e-3
        else:
            assert torch.equal(a, b)
    for l in (0, 10, 37):
        o_ref, dx_ref, g_ref = case.oracle(l)
        assert_close(case.expert_rows(out, l), o_ref, case.dtype, f"out {l}")
        assert_close(case.expert_rows(dx, l), dx_ref, case.dtype, f"dx {l}")
        for got, ref in zip(grads, g_ref):
            assert_close(got[l], ref, case.dtype, f"grad {l}")
    assert (grads[0][3] == 0).all() and (grads[2][3] == 0).all()


@pytest.mark.parametrize("backend,dtype", [(2, torch.bfloat16), (3, torch.bfloat16), (4, torch.bfloat16),
                                           (1, torch.bfloat16), (0, torch.float32)],
                         ids=["tcgen05_one_cta", "tcgen05_cta_pair", "tcgen05_panel", "cuda_cores_bf16",
                              "cuda_cores_fp32"])
def test_ffn_tanh_gelu_derivative(backend, dtype):
    """The reference's shipped backward: ``USE_MOLE_GELU`` is defined (MOLE/cpp/define.hpp:6), so
    dX1 is multiplied by the tanh-approximation derivative of MOLE/cpp/gelu.cu:3-14 while the
    forward stays the exact GELU.  Checked on every back end against the oracle run with the same
    flag; the pre-activations are spread widely enough that the two derivatives differ by far more
    than the tolerance, so a kernel that ignored the flag would fail."""
    case = Case(M=256, F=512, L=8, n_src=1, Cs=256, counts=RAGGED, dtype=dtype, seed=11,
                gelu_bwd="tanh")
    out, dx, grads = run_gpu(case, backend=backend)
    check(case, out, dx, grads, range(8), wscale=4.0 if dtype == torch.float32 else 1.0)
    exact = Case(M=256, F=512, L=8, n_src=1, Cs=256, counts=RAGGED, dtype=dtype, seed=11)
    _, dx_exact, _ = run_gpu(exact, backend=backend)
    l = 6                                        # 256 rows
    a, b = case.expert_rows(dx, l).float(), case.expert_rows(dx_exact, l).float()
    assert (a - b).abs().max() > 0, "tanh and exact derivative produced identical dx"


def test_ffn_bf16_config3_shape_spot_check():
    """The headline benchmark's shape on one GPU: M = 2048, F = 8192, 256 +- 16 rows per expert
    (capacity 320, stride 384), eight experts: tcgen05 path (one-CTA kernel, what the benchmark
    runs at this shape, and CTA pairs) against the oracle on experts with a ragged third tile,
    exactly two tiles, and the fullest one."""
    g = torch.Generator().manual_seed(9)
    L, M, F, Cs = 8, 2048, 8192, 384
    counts = torch.randint(240, 273, (L,), generator=g).tolist()
    counts[1], counts[4], counts[6] = 256, 320, 257
    case = Case(M, F, L, 1, Cs, counts, torch.bfloat16, seed=10)
    out, dx, grads = run_gpu(case)                       # backend 0: panel + resident-operand kernels here
    out3, dx3, grads3 = run_gpu(case, backend=3)
    out4, dx4, grads4 = run_gpu(case, backend=4)         # panels of 16-row granularity
    valid = torch.zeros(1, L, Cs, dtype=torch.bool)
    for l in range(L):
        valid[0, l, :counts[l]] = True
    assert torch.equal(out[valid], out3[valid]) and torch.equal(dx[valid], dx3[valid])
    assert torch.equal(out[valid], out4[valid]) and torch.equal(dx[valid], dx4[valid])
    for i, (a, b, c4) in enumerate(zip(grads, grads3, grads4)):
        assert torch.equal(a, c4)
        if i == 1:      # FC1 bias gradient: summed in the panel kernel's dX2 epilogue, in another order
            assert rel_fro(a, b) < 2e-3
        else:
            assert torch.equal(a, b)
    for l in (1, 4, 6):
        o_ref, dx_ref, g_ref = case.oracle(l)
        assert_close(case.expert_rows(out, l), o_ref, case.dtype, f"out {l}")
        assert_close(case.expert_rows(dx, l), dx_ref, case.dtype, f"dx {l}")
        for got, ref in zip(grads, g_ref):
            assert_close(got[l], ref, case.dtype, f"grad {l}")


@pytest.mark.parametrize("backend", [2, 3, 4])
def test_ffn_bf16_rows_packed_by_the_senders(backend):
    """``desc.compact = 3``: x and dout arrive already packed -- expert l's rows of all four source
    ranks in source order at the front of its run ``[l][n_src * Cs]``, pad rows holding garbage --
    as the packed form of the push-style dispatch leaves them.  The call gathers nothing, zeroes
    the pad rows in place and scatters out / dx back to the (source, expert) chunks; results must
    equal the same call on chunked inputs bit for bit (same packed layout inside) and the oracle."""
    from mole_b200 import ops
    counts = [100, 0, 256, 1, 7, 128,
              30, 0, 129, 0, 250, 128,
              0, 0, 5, 200, 255, 128,
              127, 0, 1, 56, 3, 128]            # [n_src=4][L=6]
    case = Case(M=256, F=512, L=6, n_src=4, Cs=256, counts=counts, dtype=torch.bfloat16, seed=7)
    out_c, dx_c, grads_c = run_gpu(case, backend=backend)          # chunked inputs, packed by the call
    c = case
    dev = torch.device("cuda")
    run = c.n_src * c.Cs
    xp = torch.full((c.L, run, c.M), float("nan"), dtype=c.dtype)
    dp = torch.full((c.L, run, c.M), float("nan"), dtype=c.dtype)
    for l in range(c.L):
        xp[l, :c.expert_rows(c.x, l).shape[0]] = c.expert_rows(c.x, l)
        dp[l, :c.expert_rows(c.dout, l).shape[0]] = c.expert_rows(c.dout, l)
    desc = ops.make_ffn_desc(c.dtype, c.act, "exact", c.M, c.F, c.L, c.n_src, c.Cs, 0, c.L, c.L,
                             False, backend, compact=3)
    ws = ops.ffn_workspace(desc, dev)
    rows = c.L * run
    x, dout = xp.view(rows, c.M).cuda(), dp.view(rows, c.M).cuda()
    w1, b1, w2, b2 = (t.cuda() for t in (c.w1, c.b1, c.w2, c.b2))
    nan = float("nan")
    x1 = torch.full((rows, c.F), nan, dtype=c.dtype, device=dev)
    h = torch.full((rows, c.F), nan, dtype=c.dtype, device=dev)
    out = torch.full((rows, c.M), nan, dtype=c.dtype, device=dev)
    cnt = c.counts.flatten().cuda()
    ops.ffn_fwd(desc, cnt, x, w1, b1, w2, b2, x1, h, out, ws)
    dx1 = torch.full((rows, c.F), nan, dtype=c.dtype, device=dev)
    dx = torch.full((rows, c.M), nan, dtype=c.dtype, device=dev)
    grads = [torch.full_like(t, nan) for t in (w1, b1, w2, b2)]
    ops.ffn_bwd(desc, cnt, dout, x, x1, h, w1, w2, dx1, dx, grads[0], grads[1], grads[2], grads[3], ws)
    assert ops.device_fault() == 0
    torch.cuda.synchronize()
    shape = (c.n_src, c.L, c.Cs)
    out, dx = out.view(*shape, c.M).cpu(), dx.view(*shape, c.M).cpu()
    for l in range(c.L):
        assert torch.equal(c.expert_rows(out, l), c.expert_rows(out_c, l)), f"out {l}"
        assert torch.equal(c.expert_rows(dx, l), c.expert_rows(dx_c, l)), f"dx {l}"
    for a, b in zip(grads, grads_c):
        assert torch.equal(a.cpu(), b)
    check(case, out, dx, [g.cpu() for g in grads], range(c.L))
