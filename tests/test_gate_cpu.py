"""The determinism gate, end to end on the tiny CPU model (every case must match the cold reference)."""
from vade_b200.cli.gate import run_gate
from vade_b200.config import tiny_config
from vade_b200.runtime.build import build_engine


def test_determinism_gate_passes_on_the_tiny_model():
    eng = build_engine(tiny_config(), device="cpu", seed=0, slots=17, max_seq=512, prefill_chunk=256)
    lines = []
    assert run_gate(eng, tokens=6, prompt_len=100, out=lines.append), "\n".join(lines)
    assert sum(" ok " in l for l in lines) >= 12
