"""CPU oracle for the GPT-J forward / eval-loss / decode / sampling path.

TEST INFRASTRUCTURE ONLY.  Nothing under this folder is part of the product:
only the test-suite, the smoke check and the CPU-baseline / reference arm of
the benchmark may import it, and only as the checker or the timed CPU arm.

Parity status: PARITY UNPINNED against the reference's own tests -- the
reference (kingoflolz/mesh-transformer-jax) ships no tests, golden vectors or
fixtures for this path, and its JAX/Haiku code cannot be imported in an
environment without jax.  The restatement is instead cross-checked against an
independent implementation of the same architecture (transformers'
GPTJForCausalLM, weights mapped the way the reference's to_hf_weights.py maps
them) and against itself under different shard counts.
"""
