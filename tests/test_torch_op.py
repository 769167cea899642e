"""The PyTorch operator ``aster_b200::gemm_nt``: registration, shape inference and argument
checks without a GPU; the GPU cases compare with ``torch.matmul`` in fp32 on the same inputs
(tolerance: the bf16/fp32 accumulation bound used by the other GEMM parity tests)."""

import pytest
import torch

import aster_b200.torch_op as top


def test_registered_and_fake_shapes():
    assert hasattr(torch.ops.aster_b200, "gemm_nt")
    a = torch.empty(48, 64, dtype=torch.bfloat16, device="meta")
    b = torch.empty(80, 64, dtype=torch.bfloat16, device="meta")
    c = torch.ops.aster_b200.gemm_nt(a, b, None, False, torch.bfloat16)
    assert c.shape == (48, 80) and c.dtype == torch.bfloat16 and c.device.type == "meta"
    assert torch.ops.aster_b200.gemm_nt(a, b).dtype == torch.float32


def test_cpu_tensors_are_refused():
    a = torch.zeros(16, 32, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        torch.ops.aster_b200.gemm_nt(a, a)


@pytest.mark.gpu
class TestOnGpu:
    @pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
    @pytest.mark.parametrize("shape", [(256, 512, 384), (100, 72, 264), (1024, 1024, 1024)])
    def test_matches_matmul(self, gpu, dtype, shape):
        M, N, K = shape
        g = torch.Generator(device="cuda").manual_seed(M + N + K)
        a = torch.randn(M, K, device="cuda", generator=g).to(dtype)
        b = torch.randn(N, K, device="cuda", generator=g).to(dtype)
        c = torch.ops.aster_b200.gemm_nt(a, b)
        ref = a.float() @ b.float().T
        # fp32 accumulation in a different order: K * eps_f32 * |a||b| bounds the difference
        tol = 1e-6 * K * float(a.float().abs().max() * b.float().abs().max())
        assert c.dtype == torch.float32 and float((c - ref).abs().max()) <= tol

    def test_fused_epilogue_and_stream(self, gpu):
        M, N, K = 512, 768, 256
        g = torch.Generator(device="cuda").manual_seed(7)
        a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
        bias = torch.randn(N, device="cuda", generator=g)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # the op must enqueue on torch's current stream
            c = torch.ops.aster_b200.gemm_nt(a, b, bias, True, torch.bfloat16)
        side.synchronize()
        ref = torch.relu(a.float() @ b.float().T + bias)
        err = (c.float() - ref).abs()
        # one bf16 rounding of the result (2^-8 relative) plus the accumulation slack
        bound = ref.abs() * 2.0 ** -8 + 1e-6 * K * float(a.float().abs().max() * b.float().abs().max())
        assert c.dtype == torch.bfloat16 and bool((err <= bound).all())

    def test_fp8_with_scales(self, gpu):
        M, N, K = 256, 256, 512
        g = torch.Generator(device="cuda").manual_seed(11)
        a = torch.randn(M, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
        b = torch.randn(N, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
        sa = torch.tensor([0.5], device="cuda")
        sb = torch.tensor([0.25], device="cuda")
        c = torch.ops.aster_b200.gemm_nt(a, b, None, False, torch.float32, sa, sb)
        ref = (a.float() @ b.float().T) * 0.125
        tol = 1e-6 * K * float(a.float().abs().max() * b.float().abs().max())
        assert float((c - ref).abs().max()) <= tol

    def test_direct_function_equals_the_operator(self, gpu):
        a = torch.randn(300, 520, device="cuda").bfloat16()
        b = torch.randn(200, 520, device="cuda").bfloat16()
        bias = torch.randn(200, device="cuda")
        x = torch.ops.aster_b200.gemm_nt(a, b, bias, True, torch.bfloat16)
        y = top.gemm_nt_direct(a, b, bias, True, torch.bfloat16)
        assert torch.equal(x, y)

    def test_plan_cache_reuse(self, gpu):
        top.clear_plan_cache()
        a = torch.ones(128, 64, device="cuda", dtype=torch.float16)
        for _ in range(3):
            c = torch.ops.aster_b200.gemm_nt(a, a)
        assert len(top._plans) == 1 and float(c[0, 0]) == 64.0
        top.clear_plan_cache()

    def test_cuda_graph_replays(self, gpu):
        """A launch recorded into a CUDA graph and replayed on new data equals the eager launch
        bit for bit -- also for a plan whose last tiles are cut along K, whose ready flags are
        versioned per launch (a replay reuses the recorded version, so each replay clears the
        flags first)."""
        # the last shape: a skinny problem whose K ranges meet in a CTA cluster's shared memory
        for M, N, K in [(512, 512, 2048), (384, 640, 256), (16, 1024, 4096)]:
            g = torch.Generator(device="cuda").manual_seed(M + K)
            a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
            b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
            torch.ops.aster_b200.gemm_nt(a, b, None, False, torch.bfloat16)  # builds the plan outside the capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                c = torch.ops.aster_b200.gemm_nt(a, b, None, False, torch.bfloat16)
            for seed in range(3):
                fresh = torch.randn(M, K, device="cuda", generator=g).bfloat16()
                a.copy_(fresh)
                graph.replay()
                torch.cuda.synchronize()
                eager = torch.ops.aster_b200.gemm_nt(fresh, b, None, False, torch.bfloat16)
                assert torch.equal(c, eager), (M, N, K, seed)
