"""Validates tests/golden/jax_stand_in by running the REFERENCE'S OWN test files on it.

    python tests/golden/run_reference_tests_on_stand_in.py /path/to/jaxmodules-checkout

tests/test_mapped_attention.py (51 tests: masked_attention_via_map and its gradients against torch's
scaled_dot_product_attention), tests/test_block_mask.py (10: the literal known answers), tests/test_attention.py
(9: flex_attention against torch FlexAttention) and tests/test_vectorize.py (23) of acutkosky/jaxmodules all pass; the
vectors of make_reference_vectors.py come from the same sources on the same stand-in.  Nothing is written into the
checkout (no bytecode, no pytest cache)."""
import os
import subprocess
import sys
import tempfile
from pathlib import Path

FILES = ["test_mapped_attention.py", "test_block_mask.py", "test_attention.py", "test_vectorize.py"]


def main(checkout: str) -> int:
    here = Path(__file__).resolve().parent
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1",
               PYTHONPATH=os.pathsep.join([str(here / "jax_stand_in"), checkout]))
    tests = [str(Path(checkout) / "tests" / f) for f in FILES]
    with tempfile.TemporaryDirectory() as cwd:
        return subprocess.call([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", *tests], env=env, cwd=cwd)


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
