from mindspeed_b200.utils.patterns import match


def test_segment_aware_patterns():
    assert match("layers.0.up", "layers.*.up")
    assert not match("layers.0.moe.experts.1.up", "layers.*.up")          # '*' stays inside one dotted segment
    assert match("layers.0.moe.experts.1.up", "layers.**.up")             # '**' crosses segments
    assert match("layers.0.moe.experts.3", "**.experts.*") and not match("layers.0.moe.experts.3.up", "**.experts.*")
    assert match("embed", "embed") and not match("embed2", "embed") and match("embed2", "embed?")
    assert not match("a.b", "a?b")                                        # '?' never matches the separator
