"""Host-side choices that need no GPU: which launches a step asks for."""
from metallix_b200 import ops


def test_key_shares_of_the_prompt_kernel():
    # enough (tile, head) blocks, or few keys: one block per tile and head
    assert ops.flash_key_shares(256, 8192) == 1
    assert ops.flash_key_shares(16, 2047) == 1
    assert ops.flash_key_shares(16, 0) == 1                 # no bound known: taken as few
    # few blocks, many keys: shares of at least 1,024 keys, at most 8, at most what fills 148 SMs
    assert ops.flash_key_shares(64, 4096) == 2
    assert ops.flash_key_shares(16, 4096) == 4
    assert ops.flash_key_shares(16, 40960) == 8
    assert ops.flash_key_shares(48, 40960) == 3
    # a window bounds the keys a tile sees
    assert ops.flash_key_shares(16, 40960, window=1024) == 1
    assert ops.flash_key_shares(16, 40960, window=4096) == 4
    try:
        ops.KEY_SHARES = 5
        assert ops.flash_key_shares(256, 10) == 5
    finally:
        ops.KEY_SHARES = None


def test_thresholds_are_ordered():
    from metallix_b200.engine import engine
    from metallix_b200.parts import feed_forward
    assert ops.SKINNY_ROWS < feed_forward.FUSED_ACTIVATION_ROWS
    assert engine.LONG_CONTEXT % engine.WIDE_TILE == 0 and engine.LONG_CONTEXT <= engine.STEP_GRAPH_TOKENS
