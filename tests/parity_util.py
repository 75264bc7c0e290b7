"""Helpers shared by the GPU parity tests (they live with the oracle: oracle/parity_checks.py)."""

from oracle.parity_checks import (BF16, MAX_ABS, REL_L2, big_lora, big_weight, check_mlp_layer,  # noqa: F401
                                  check_projection_chain, device_normal, sample_rows, small_batch_accumulator, to_dev,
                                  to_np, uniform_ids)
