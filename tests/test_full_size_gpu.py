"""Full-size parity of the headline configuration in one process (opt-in: B200_FULL_SIZE=1, several
minutes of host time for the fp32 oracle on the machine that holds the GPU): Llama-3.1-8B
architecture, 32 layers, 8192-token prompt, 32 greedy decode steps, against the layer-streamed fp32
CPU oracle with the same seeded weights.  The same check for all five benchmark configurations,
split into a short GPU half and a host half, is tests/full_size/dump_gpu.py + compare_cpu.py.
Tolerances as in tests/test_decoder_gpu.py (per-layer hidden states 2e-2, logits cosine 0.999,
greedy tokens by teacher forcing with the near-tie rule), except that below the first few layers
the hidden-state and cosine bounds widen to 1.25x / 1.5x the distance the reference's own bf16
eager numerics (second oracle pass) have from fp32 at that depth."""
import os

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(os.environ.get("B200_FULL_SIZE") != "1", reason="set B200_FULL_SIZE=1 (slow)")
def test_llama31_8b_8k_prompt(dev):
    from hoid_optimized_models_b200.configs import LLAMA31_8B
    from tests.test_decoder_gpu import _run
    cos_min, margin_min, flips = _run(dev, LLAMA31_8B, P=8192, seed=2, bf16_floor=True)
    print(f"full-size Llama-3.1-8B @8192: min logit cosine {cos_min:.6f}, min oracle top-2 margin "
          f"{margin_min:.4f}, near-tie flips at steps {flips}")
