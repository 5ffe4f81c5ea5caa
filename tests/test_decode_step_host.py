"""Host-side checks of the captured serving step: it refuses to exist without a GPU."""

import pytest
import torch


def test_captured_step_has_no_cpu_path():
    from attnarc_b200.decode_step import CapturedDecodeStep

    kv_cache = torch.zeros((4, 2, 16, 2, 128), dtype=torch.bfloat16)
    cos_sin = torch.zeros((64, 128), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        CapturedDecodeStep(kv_cache, cos_sin, sequences=2, query_heads=4, max_blocks_per_sequence=4,
                           max_sequence_length=64, dtype=torch.bfloat16)
