"""Config 1: tiny hybrid MoE in fp32 on CPU: plumbing + determinism."""
import torch

from vade_b200.config import tiny_config
from vade_b200.runtime.build import build_engine


def _prompt(n=128, vocab=4096, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab - 8, (n,), generator=g).tolist()


def _run(draft=0, n_new=64, chunk=2048, n_prompt=128):
    cfg = tiny_config()
    eng = build_engine(cfg, seed=0, prefill_chunk=chunk, max_seq=512)
    seq = eng.generate(_prompt(n_prompt), n_new, draft_depth=draft)
    return seq


def test_two_runs_identical():
    a = _run().generated
    b = _run().generated
    assert len(a) == 64 and a == b


def test_prompt_chunking_invariant():
    a = _run(n_new=16).generated
    b = _run(n_new=16, chunk=64).generated
    assert a == b


def test_speculative_identical():
    a = _run(n_new=32)
    b = _run(n_new=32, draft=3)
    assert a.generated == b.generated
    assert b.drafted > 0
