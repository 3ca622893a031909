"""The reference's own test suite (``tests/test_correctness.py``), restated against this package
under the reference's import name: same classes of checks, shapes, seed, hyper-parameters and
tolerances.  Inputs are drawn on the CPU (the reference draws them on the GPU; its seed-42 CUDA
stream is not reproducible on a CPU oracle) and the expected values come from the torch restatement
of its ``_reference_*`` helpers in ``oracle.torch_steps``."""

import pytest
import torch

from oracle import torch_steps as T

pytestmark = pytest.mark.gpu

ATOL = RTOL = 5e-3      # reference tolerance for its TF32 dot (test_correctness.py:21-24)
QATOL = QRTOL = 0.05    # reference tolerance with int8 moments (:134-136)
SHAPES = [(128, 256, 128), (64, 512, 256), (256, 1024, 512)]


def _inputs(BT, V, H):
    torch.manual_seed(42)
    go, inp, w = torch.randn(BT, V), torch.randn(BT, H), torch.randn(V, H)
    m, v = torch.randn(V, H) * 0.01, torch.randn(V, H).abs() * 0.01
    return go, inp, w, m, v


class TestFusedGradSGD:
    @pytest.mark.parametrize("BT,V,H", SHAPES)
    def test_matches_reference(self, BT, V, H):
        from fused_grad_optimizer.kernel import fused_grad_sgd
        go, inp, w, _, _ = _inputs(BT, V, H)
        expect = T.sgd_step(go, inp, w, 0.01, 0.1)
        wf = w.cuda()
        fused_grad_sgd(go.cuda(), inp.cuda(), wf, lr=0.01, weight_decay=0.1)
        torch.testing.assert_close(wf.cpu(), expect, atol=ATOL, rtol=RTOL)


class TestFusedGradAdamW:
    @pytest.mark.parametrize("BT,V,H", SHAPES)
    def test_matches_reference(self, BT, V, H):
        from fused_grad_optimizer.kernel import fused_grad_adamw
        go, inp, w, m, v = _inputs(BT, V, H)
        ew, em, ev = T.adamw_step(go, inp, w, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 5)
        wf, mf, vf = w.cuda(), m.cuda(), v.cuda()
        fused_grad_adamw(go.cuda(), inp.cuda(), wf, mf, vf, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8,
                         weight_decay=0.01, step=5)
        torch.testing.assert_close(wf.cpu(), ew, atol=ATOL, rtol=RTOL)
        torch.testing.assert_close(mf.cpu(), em, atol=ATOL, rtol=RTOL)
        torch.testing.assert_close(vf.cpu(), ev, atol=ATOL, rtol=RTOL)

    def test_bf16_weight(self):
        from fused_grad_optimizer.kernel import fused_grad_adamw
        torch.manual_seed(42)
        BT, V, H = 128, 256, 128
        go = torch.randn(BT, V, dtype=torch.bfloat16).cuda()
        inp = torch.randn(BT, H, dtype=torch.bfloat16).cuda()
        w = torch.randn(V, H, dtype=torch.bfloat16).cuda()
        m, v = torch.zeros(V, H, device="cuda"), torch.zeros(V, H, device="cuda")
        before = w.clone()
        fused_grad_adamw(go, inp, w, m, v, step=1)
        assert not torch.equal(w, before)


class TestFusedGradAdamWInt8State:
    @pytest.mark.parametrize("BT,V,H", SHAPES)
    def test_matches_reference(self, BT, V, H):
        from fused_grad_optimizer.kernel import fused_grad_adamw_int8state
        go, inp, w, m, v = _inputs(BT, V, H)
        ew, _, _ = T.adamw_step(go, inp, w, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 5)
        mq, ms = T.int8_quantise(m, 64)
        vq, vs = T.int8_quantise(v, 64)
        wf = w.cuda()
        fused_grad_adamw_int8state(go.cuda(), inp.cuda(), wf, mq.cuda(), vq.cuda(), ms.cuda(), vs.cuda(),
                                   lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=5, qblock=64)
        torch.testing.assert_close(wf.cpu(), ew, atol=QATOL, rtol=QRTOL)

    def test_bf16_weight(self):
        from fused_grad_optimizer.kernel import fused_grad_adamw_int8state
        torch.manual_seed(42)
        BT, V, H = 128, 256, 128
        go = torch.randn(BT, V, dtype=torch.bfloat16).cuda()
        inp = torch.randn(BT, H, dtype=torch.bfloat16).cuda()
        w = torch.randn(V, H, dtype=torch.bfloat16).cuda()
        mq, vq = torch.zeros(V, H, dtype=torch.int8, device="cuda"), torch.zeros(V, H, dtype=torch.int8, device="cuda")
        ms, vs = torch.ones(V, H // 64, device="cuda"), torch.ones(V, H // 64, device="cuda")
        before = w.clone()
        fused_grad_adamw_int8state(go, inp, w, mq, vq, ms, vs, step=1, qblock=64)
        assert not torch.equal(w, before)
        assert mq.any()


class TestFusedLinearQuantized:
    def test_forward_backward_quantized(self):
        from fused_grad_optimizer.module import FusedLinear
        torch.manual_seed(42)
        layer = FusedLinear(128, 64, optimizer_type="adamw", quantize_state=True).cuda()
        layer.train()
        layer.update_optimizer_config(lr=1e-3, step=1, weight_decay=0.01)
        x = torch.randn(8, 128, device="cuda", requires_grad=True)
        before = layer.weight.data.clone()
        layer(x).sum().backward()
        assert not torch.equal(layer.weight.data, before)
        assert x.grad is not None
        assert layer._state.m_q is not None and layer._state.m_q.dtype == torch.int8
        assert layer.weight.grad is None

    def test_memory_savings(self):
        from fused_grad_optimizer.module import FusedLinear
        V, H = 1024, 512
        sizes = []
        for q in (False, True):
            layer = FusedLinear(H, V, optimizer_type="adamw", quantize_state=q).cuda()
            layer.train()
            layer.update_optimizer_config(lr=1e-3, step=1)
            layer._ensure_state()
            layer._state.ensure_buffers()
            st = layer._state
            sizes.append(st.m_q.nbytes + st.v_q.nbytes + st.m_scale.nbytes + st.v_scale.nbytes if q
                         else st.m.nbytes + st.v.nbytes)
        assert sizes[1] < sizes[0]


class TestFusedLinearModule:
    def test_forward_backward(self):
        from fused_grad_optimizer.module import FusedLinear
        torch.manual_seed(42)
        layer = FusedLinear(128, 64, optimizer_type="adamw").cuda()
        layer.train()
        layer.update_optimizer_config(lr=1e-3, step=1, weight_decay=0.01)
        x = torch.randn(8, 128, device="cuda", requires_grad=True)
        before = layer.weight.data.clone()
        layer(x).sum().backward()
        assert not torch.equal(layer.weight.data, before)
        assert x.grad is not None

    def test_eval_mode_no_update(self):
        from fused_grad_optimizer.module import FusedLinear
        layer = FusedLinear(128, 64, optimizer_type="adamw").cuda()
        layer.eval()
        assert layer(torch.randn(8, 128, device="cuda")).shape == (8, 64)

    def test_from_linear(self):
        from fused_grad_optimizer.module import FusedLinear
        original = torch.nn.Linear(128, 64, bias=False).cuda()
        fused = FusedLinear.from_linear(original, optimizer_type="adamw")
        assert torch.equal(fused.weight.data, original.weight.data)
        assert fused.weight.data_ptr() == original.weight.data_ptr()


class TestFusedOptimizerManager:
    def test_excludes_fused_params(self):
        from fused_grad_optimizer.module import FusedLinear, FusedOptimizerManager
        model = torch.nn.Sequential(torch.nn.Linear(128, 64), torch.nn.ReLU(),
                                    FusedLinear(64, 32, optimizer_type="adamw")).cuda()
        manager = FusedOptimizerManager(model)
        non_fused = {id(p) for p in manager.get_non_fused_params()}
        assert id(model[2].weight) in manager._fused_param_ids
        assert id(model[2].weight) not in non_fused
        assert id(model[0].weight) in non_fused
