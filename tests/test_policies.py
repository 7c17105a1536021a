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
    from metallix_b200.parts import attention, feed_forward
    assert ops.SKINNY_ROWS < feed_forward.FUSED_ACTIVATION_ROWS
    assert attention.LONG_CONTEXT % attention.WIDE_TOKENS == 0 and attention.LONG_CONTEXT <= engine.STEP_GRAPH_TOKENS
    assert attention.WIDE_TOKENS % attention.TILE_TOKENS == 0


def test_the_attention_prepares_its_own_tile_lists():
    """Portions become tiles of 16 and of 128 tokens (those with most keys
    first), single tokens decode rows; padding rows of a graph bring nothing;
    what a replayed step is launched with is the bound, not the step's own."""
    from metallix_b200.parts import StepPlan
    from metallix_b200.parts.attention import attention_tiles
    made = attention_tiles(StepPlan([5, 1, 300, 1], [0, 7, 2000, 0], 4, 2300))
    tiles = {name: array.tolist() for name, array in made.arrays.items()}
    assert tiles["tile_request"] == [0] + [2] * 19 + [1, 3] and made.facts["multi_tiles"] == 20
    assert tiles["tile_start"][:3] == [0, 6, 22] and tiles["tile_length"][19:] == [12, 1, 1]
    assert tiles["decode_token"] == [5, 306] and tiles["decode_request"] == [1, 3]
    assert tiles["wide_request"] == [2, 2, 2, 0] and tiles["wide_start"] == [262, 134, 6, 0]
    assert tiles["wide_length"] == [44, 128, 128, 5]
    assert made.facts["longest_context"] == 8 and made.facts["longest_keys"] == 2300 and made.graph_key is True
    again = attention_tiles(StepPlan([5, 1, 300, 1], [0, 7, 2000, 0], 4, 4096, replayable=True))
    assert again.facts["longest_context"] == 4096 and again.facts["longest_keys"] == 4096
    assert all(array.shape == made.arrays[name].shape for name, array in again.arrays.items())
    short = attention_tiles(StepPlan([40], [100], 1, 2048, replayable=True))
    assert short.graph_key is False and short.facts["longest_keys"] == 2047
    graph = attention_tiles(StepPlan([1, 1, 1, 1], None, 2, 4096, replayable=True))
    assert graph.arrays["tile_length"].tolist() == [1, 1, 0, 0]
    assert graph.arrays["decode_token"].tolist() == [0, 1, -1, -1] and graph.facts["longest_context"] == 4096
