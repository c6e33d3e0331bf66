"""Host-side rules of the decode overlap (no GPU): when the next step may be launched ahead of the text work,
and how a pre-launched step is recognised."""
from types import SimpleNamespace

from tgi_b200.models.flash_causal_lm import FlashCausalLM
from tgi_b200.utils.tokens import StopSequenceCriteria, StoppingCriteria


def _seq(n_ids, max_new, done, eos=(2,), ignore_eos=False, stops=(), n_slots=64):
    st = StoppingCriteria(set(eos), [StopSequenceCriteria(s) for s in stops], max_new, ignore_eos)
    st.current_tokens = done
    return SimpleNamespace(ids=list(range(n_ids)), stopping=st, slots=list(range(n_slots)))


def test_nobody_finishes_rules():
    ok = FlashCausalLM._nobody_finishes
    a, b = _seq(10, 20, 3), _seq(12, 20, 5)
    assert ok([a, b], [7, 9])
    assert not ok([a, b], [7, 2])                                   # EOS for the second sequence
    assert ok([a, _seq(12, 20, 5, ignore_eos=True)], [7, 2])        # ... unless it ignores EOS
    assert not ok([a, _seq(12, 6, 5)], [7, 9])                      # reaches max_new_tokens with this token
    assert not ok([a, _seq(12, 20, 5, stops=("\n\n",))], [7, 9])    # stop strings need the text
    assert not ok([a, _seq(63, 200, 5, n_slots=64)], [7, 9])        # no slot left for the step after
    assert ok([a, _seq(62, 200, 5, n_slots=64)], [7, 9])


def test_decode_signature_tracks_identity_and_length():
    sig, same = FlashCausalLM._decode_signature, FlashCausalLM._same_step
    a, b = _seq(10, 20, 3), _seq(12, 20, 5)
    s0 = sig([a, b])
    assert same(s0, [a, b]) and not same(s0, [b, a]) and not same(s0, [a])
    # an equal-looking but different sequence object is a different step
    assert not same(s0, [a, _seq(12, 20, 5)])
    a.ids.append(1)
    assert not same(s0, [a, b]) and same(sig([a, b]), [a, b])
