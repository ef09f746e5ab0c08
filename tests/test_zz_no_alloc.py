"""``dionw_newton_schulz_static``: the orthogonalization for callers that cannot allocate.

Some users of this library have no allocator to ask for the iteration's scratch: a C host
bound to the ABI without torch, a serving loop with a memory budget fixed at start-up, a
process whose device memory already sits in a framework's pool.  For them the library
carries a fixed 64 MiB scratch of its own.  This file checks, through the C ABI, that the
entry point gives the same bits as the ordinary one (it runs the same products on other
scratch memory, so the tolerance of the other tests, rel-L2 2e-3, is met with 0), twice in
a row (the second call starts from the first call's leftovers), and that a problem beyond
the ceiling is refused.  It is collected last so that a failure here cannot hide another.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _operand(blocks: int, m: int, n: int, seed: int) -> torch.Tensor:
    x = torch.randn(blocks, m, n, generator=torch.Generator().manual_seed(seed))
    x = x / (torch.linalg.vector_norm(x, dim=(-2, -1), keepdim=True) + 1e-8)
    return x.half().to(DEV)


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm())


def test_static_scratch_entry_matches_the_workspace_entry_twice() -> None:
    """Two calls in a row (the second starts from the first one's leftovers), then the other
    layouts of the scratch: a square block (standard iteration) and the bf16 kinds."""
    from dionw_b200 import _native

    _native.library()
    cases = [(2, 512, 2048, _native.NS_GRAM), (3, 256, 1024, _native.NS_GRAM), (2, 640, 640, _native.NS_GRAM),
             (2, 384, 1000, _native.NS_POLAR_EXPRESS), (1, 512, 512, _native.NS_KELLER)]
    for call, (blocks, m, n, kind) in enumerate(cases):
        x = _operand(blocks, m, n, seed=call)
        if kind != _native.NS_GRAM:
            x = x.bfloat16()
        need = _native.newton_schulz_workspace_bytes(blocks, m, n, kind)
        assert 0 < need <= _native.STATIC_SCRATCH_BYTES
        expect = torch.empty(blocks, m, n, dtype=torch.bfloat16, device=DEV)
        workspace = torch.empty(need, dtype=torch.uint8, device=DEV)
        _native.newton_schulz(x.clone(), expect, m, n, kind, workspace)
        got = torch.empty(blocks, m, n, dtype=torch.bfloat16, device=DEV)
        operand = x.clone()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        _native.newton_schulz_static(operand, got, m, n, kind)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert _native.device_status() == 0
        assert _rel(got.float(), expect.float()) <= 2e-3
        assert torch.equal(got, expect)
        # nothing was allocated: not through torch, and not from the driver behind its back
        # (the first call may be the one that loads the library's device image, scratch included)
        assert torch.cuda.memory_allocated() == before
        if call > 0:
            assert free_after >= free_before


def test_static_scratch_entry_refuses_problems_beyond_its_ceiling() -> None:
    from dionw_b200 import _native

    blocks, m, n = 8, 1024, 4096
    assert _native.newton_schulz_workspace_bytes(blocks, m, n, _native.NS_GRAM) > _native.STATIC_SCRATCH_BYTES
    x = torch.zeros(blocks, m, n, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="built-in scratch holds"):
        _native.newton_schulz_static(x, x.view(torch.bfloat16), m, n, _native.NS_GRAM)


def test_static_scratch_entry_refuses_padded_operands() -> None:
    """The ceiling is stated for the smallest legal leading dimension; a wider one is refused by this
    entry itself, with a message that names the built-in scratch."""
    from dionw_b200 import _native

    blocks, m, n = 1, 256, 1000
    x = torch.zeros(blocks, m, 1024, dtype=torch.float16, device=DEV)[..., :1016]   # ldx = 1024, not 1000
    with pytest.raises(ValueError, match="built-in"):
        _native.newton_schulz_static(x, torch.empty(blocks, m, 1024, dtype=torch.bfloat16, device=DEV), m, n,
                                     _native.NS_GRAM)
