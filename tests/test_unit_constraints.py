"""Constraint state machines of the sampler loop: stop-sequence automaton with hold-back, forced tokens, JSON close
forcing, thinking budget."""
import json
import random

from hipengine_b200.generation.constraints import (ForcedTokenQueue, JsonObjectConstraintState, ThinkingBudgetState,
                                                   TokenSequenceDFAState, json_closing_suffix)


def test_stop_sequence_automaton_matches_and_holds_back():
    d = TokenSequenceDFAState([(5, 6, 7), (9,), ()])
    assert not d.push(1) and d.holdback() == 0
    assert not d.push(5) and d.holdback() == 1            # could become 5 6 7
    assert not d.push(6) and d.holdback() == 2
    assert not d.push(5) and d.holdback() == 1            # 5 6 5: only the last 5 can still start a stop
    assert not d.push(6) and not d.matched
    assert d.push(7) and d.matched == (5, 6, 7)
    e = TokenSequenceDFAState([(5, 6, 7), (9,)])
    assert e.push(9) and e.matched == (9,)
    assert not TokenSequenceDFAState([]).push(3)


def test_forced_token_queue():
    q = ForcedTokenQueue([1, 2], reason="close")
    assert q and q.pop() == 1
    q.extend([3], reason="again")
    assert [q.pop(), q.pop()] == [2, 3] and not q and q.reason == "again"


def test_thinking_budget_state():
    t = ThinkingBudgetState(close_ids=(7, 8), hard_cap=6, soft_window=3)
    assert t.thinking and t.suppress_eos() and t.close_bias() == 0.0
    for tok in (1, 2, 3):
        t.push(tok)
    assert t.close_bias() > 0 and not t.must_force_close()          # inside the soft window: 3 of 6 spent
    ramp = []
    for tok in (4, 5, 6):
        ramp.append(t.close_bias())
        t.push(tok)
    assert ramp == sorted(ramp) and ramp[-1] == 10.0 and t.must_force_close()
    assert t.forced_close() == [7, 8] and not t.thinking and not t.suppress_eos()
    u = ThinkingBudgetState(close_ids=(7, 8), hard_cap=50)
    for tok in (1, 7, 8, 9):
        u.push(tok)
    assert not u.thinking and u.n_think == 3                         # closed by the model itself after three tokens
    assert not ThinkingBudgetState().thinking                        # no close sequence: nothing to track


def test_any_prefix_of_a_json_object_can_be_closed_into_a_parseable_one():
    rng = random.Random(11)

    def value(depth):
        r = rng.random()
        if depth > 2 or r < 0.35:
            return rng.choice([True, False, None, 0, -3, 12.5, 1e-3, "", "text", 'quote " and \\\\ slash', "unicode \\u00e9"])
        if r < 0.65:
            return [value(depth + 1) for _ in range(rng.randrange(0, 4))]
        return {f"k{i}": value(depth + 1) for i in range(rng.randrange(0, 4))}

    for trial in range(40):
        doc = {f"key{i}": value(0) for i in range(rng.randrange(1, 5))}
        for text in (json.dumps(doc), json.dumps(doc, indent=1), json.dumps(doc, separators=(",", ":"))):
            for n in range(1, len(text) + 1):
                prefix = text[:n]
                closed = prefix + json_closing_suffix(prefix)
                try:
                    obj = json.loads(closed)
                except Exception as exc:                      # noqa: BLE001
                    raise AssertionError((prefix, closed, str(exc)))
                assert isinstance(obj, dict)
    assert json_closing_suffix('{"a": 1,') == ' "_": null}' and json_closing_suffix('{"a": [1,') == " null]}"
    assert json_closing_suffix('{"ab') == '": null}' and json_closing_suffix('{"a": tr') == "ue}"
    assert json_closing_suffix('{"a": -') == "0}"
    lone = '{"a": "x' + chr(92)                                # the text ends in a lone backslash
    assert json_closing_suffix(lone) == chr(92) + '"}' and json.loads(lone + json_closing_suffix(lone)) == {"a": "x" + chr(92)}
    assert json_closing_suffix('{"a": {}}') == ""


def test_json_object_state_detects_completion_and_forces_a_close():
    enc = lambda s: [ord(c) for c in s]
    dec = lambda ids: "".join(chr(i) for i in ids)
    st = JsonObjectConstraintState(dec, enc)
    assert dec(st.forced_close_tokens()) == "{}"
    for ch in '{"a": [1, 2':
        st.push(ord(ch))
    assert not st.complete and dec(st.forced_close_tokens()) == "]}"
    for ch in "]}":
        st.push(ord(ch))
    assert st.complete and dec(st.forced_close_tokens()) == ""


def test_json_mode_forces_a_parseable_close_before_the_token_budget_runs_out():
    """The scheduler's commit path with JSON close forcing, fed a scripted byte stream: however deep the nesting is
    when the budget nears its end, the forced suffix still fits and the finished text parses as an object."""
    from hipengine_b200.generation.scheduler import Scheduler
    from hipengine_b200.generation.types import GenerationRequest
    enc = lambda s: [ord(c) for c in s]
    dec = lambda ids: "".join(chr(i) for i in ids)
    scripts = ['{"k": [[[[[[1, 2, {"deep": {"er": [true, fal',
               '{"a": "a long string value that never closes by itself and keeps going and going',
               '{"list": [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21,',
               '{"x": {"y": {"z": {"w": {"v": {"u": {"t": {"s": {"r": {"q": {"p": {"o":']
    for script in scripts:
        for budget in (len(script) + 4, len(script) + 12, 40):
            sched = Scheduler(4, 16, eos_token_id=None, decode=dec, encode=enc)
            rs = sched.submit(GenerationRequest(prompt_token_ids=[1], max_tokens=budget, ignore_eos=True,
                                                json_object_close_forcing=True))
            sched.active[rs.rid] = rs
            stream = iter(enc(script) + [ord("1")] * budget)
            done = False
            while not done:
                tok = rs.forced.pop() if rs.forced else next(stream)
                done = sched.record_token(rs, tok)
            text = dec(rs.generated)
            assert len(rs.generated) <= budget
            obj = json.loads(text)
            assert isinstance(obj, dict), text
