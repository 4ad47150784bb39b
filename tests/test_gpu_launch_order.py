"""Back-to-back launches on a non-blocking stream with inputs that change every iteration and no host
synchronisation in between: each kernel starts while its predecessor still runs (programmatic dependent
launch), so every result must equal the one obtained with a synchronisation after every call.  Guards
against a kernel reading its input ahead of its dependency wait (a load through the read-only path may
be moved there by the compiler) and against stale cached activations at a reused address."""
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from tensorpencil_b200.backend import Backend
    b = Backend(0)
    yield b
    b.close()


@pytest.mark.parametrize("n,k,m", [(5120, 17408, 8), (4096, 5120, 8), (4096, 5120, 1)])
def test_gemv_sees_the_activations_of_its_own_iteration(be, n, k, m):
    from tensorpencil_b200 import harness
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        w = harness.rotating_q8_weights(n, k, 1, be.device)[0]
        xs = [torch.randn(m, k, device="cuda") * (1 + i) for i in range(4)]
        ref = []
        for x in xs:
            y = torch.empty(m, n, device="cuda")
            be.opGemvQuantizeX(x, m * k)
            be.opGemvQuantQ8N("q8_0", y, w, 1.0, n, k, m, 0, m)
            torch.cuda.synchronize()
            ref.append(y.clone())
        ys = [torch.empty(m, n, device="cuda") for _ in range(80)]
        torch.cuda.synchronize()
        for i, y in enumerate(ys):
            be.opGemvQuantizeX(xs[i % 4], m * k)
            be.opGemvQuantQ8N("q8_0", y, w, 1.0, n, k, m, 0, m)
        torch.cuda.synchronize()
    be.status_poll()
    assert all(torch.equal(y, ref[i % 4]) for i, y in enumerate(ys))


@pytest.mark.parametrize("bits", [8, 4])
def test_linear_sees_the_activations_of_its_own_iteration(be, bits):
    from tensorpencil_b200 import synth
    m, n, k = 512, 1024, 1024
    c = synth.convrot_linear(m, n, k, bits, seed=41)
    w = torch.from_numpy(c["w_packed"] if bits == 4 else c["w_i8"]).cuda()
    ws = torch.from_numpy(c["w_scale"]).cuda()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        xs = [torch.randn(m, k, device="cuda") * (1 + 3 * i) for i in range(3)]
        ref = []
        for x in xs:
            y = torch.empty(m, n, device="cuda")
            be.convrot_linear(x, w, ws, n, bits, y=y)
            torch.cuda.synchronize()
            ref.append(y.clone())
        ys = [torch.empty(m, n, device="cuda") for _ in range(60)]
        for i, y in enumerate(ys):
            be.convrot_linear(xs[i % 3], w, ws, n, bits, y=y)
        torch.cuda.synchronize()
    be.status_poll()
    assert all(torch.equal(y, ref[i % 3]) for i, y in enumerate(ys))
