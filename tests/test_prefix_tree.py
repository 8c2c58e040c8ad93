"""Prefix-tree merge rules, text-prefix matching and one-step-per-leaf training extraction."""
import torch

from axon_b200.engine.state.prefix_tree import PrefixTree
from axon_b200.engine.state.program_state import ProgramManager, ProgramState, Step, TerminationReason


def ins(t, ids, masks, step, strs=None, lps=None, rms=None):
    return t.insert(ids, strs or [f"<{i}>" for i in ids], masks, lps or [-0.1 * i for i in ids], rms, step_idx=step)


def test_insert_merge_rules():
    t = PrefixTree()
    ins(t, [1, 2, 3], [0, 0, 1], 0, strs=["a", "", "c"], rms=[[[-1, -1]], [], [[4, 5]]])
    assert t.size() == 3
    ins(t, [1, 2, 3, 4], [0, 0, 0, 1], 1, strs=["a", "b", "c", "d"], rms=[[[7, 8]], [[1, 2]], [[-1, -1]], [[9, 9]]])
    n1 = t.root.get_child(1)
    n2, n3 = n1.get_child(2), n1.get_child(2).get_child(3)
    assert n3.masks == {0, 1} and n3.step_idx == 0          # masks united, min step kept
    assert n2.token_str == "b"                              # back-filled
    assert n1.moe_routermap == [[7, 8]]                     # all -1 replaced by valid
    assert n2.moe_routermap == [[1, 2]]                     # empty replaced
    assert n3.moe_routermap == [[4, 5]]                     # valid never overwritten by -1
    assert t.longest_prefix([1, 2, 9]) == [1, 2] and t.size() == 4
    assert "ROOT" in repr(t)


def test_longest_text_prefix_prefers_longest_child():
    t = PrefixTree()
    t.insert([10, 11], ["he", "llo"], [0, 0], [0, 0])
    t.insert([12, 13], ["hel", "p"], [0, 0], [0, 0])
    ids, strs, pos, mm = t.longest_text_prefix("help me")
    assert ids == [12, 13] and pos == 4 and mm == []
    ids, _, pos, _ = t.longest_text_prefix("hello world")
    assert ids == [12] and pos == 3          # greedy: "hel" wins, then no child matches "lo"
    assert t.longest_text_prefix("xyz")[0] == []


def test_mm_expansion_skipped_as_a_unit():
    t = PrefixTree()
    t.insert([1, 99, 99, 99, 2], ["<img>", "", "", "", "ok"], [0] * 5, [0.0] * 5, mm_expansions=[(1, 3, "h1")])
    text = "<img>" + "[IMAGE]" + "ok!"
    region = (5, 12, "image", "h1", "pixels")
    ids, _, pos, rec = t.longest_text_prefix(text, [region])
    assert ids == [1, 99, 99, 99, 2] and pos == 14 and rec == [("image", "pixels")]
    ids, _, pos, _ = t.longest_text_prefix(text, [(5, 12, "image", "other", "x")])
    assert ids == [1] and pos == 5           # content changed: stop before the run


def test_one_training_step_per_leaf_and_prefix_trained_once():
    p = ProgramState(uid="u", session_id="s")
    ins(p.prefix_tree, [1, 2, 3, 4], [0, 0, 1, 1], 0)
    ins(p.prefix_tree, [1, 2, 3, 4, 5, 6], [0, 0, 0, 0, 0, 1], 1)
    ins(p.prefix_tree, [1, 2, 7, 8], [0, 0, 1, 1], 2)
    steps = sorted(p.get_training_steps(), key=lambda s: s.order_idx)
    assert [s.tokens for s in steps] == [[1, 2, 3, 4, 5, 6], [1, 2, 7, 8]]
    assert steps[0].masks == [0, 0, 1, 1, 0, 1] and steps[0].order_idx == 1
    assert steps[1].masks == [0, 0, 1, 1] and steps[1].order_idx == 2
    trained = {}
    for s in steps:
        for tok, m in zip(s.tokens, s.masks):
            trained[tok] = trained.get(tok, 0) + m
    assert all(v <= 1 for v in trained.values()) and sum(trained.values()) == 5
    p.done, p.reward = True, 1.0
    assert p.is_trainable() and not p.is_trainable(strict=True)
    p.termination_reason = TerminationReason.ENV_DONE
    assert p.is_trainable(strict=True)
    p.reward = -1e99
    assert not p.is_trainable()


def test_sibling_with_shared_generated_prefix_masks_it_in_second_leaf():
    p = ProgramState(uid="u", session_id="s")
    ins(p.prefix_tree, [1, 2, 3], [0, 1, 1], 0)
    ins(p.prefix_tree, [1, 2, 4], [0, 1, 1], 1)
    steps = {tuple(s.tokens): s for s in p.get_steps_from_prefix_tree()}
    assert steps[(1, 2, 3)].masks == [0, 1, 1]
    assert steps[(1, 2, 4)].masks == [0, 0, 1]


def test_routermap_stacking_and_step_set_response():
    p = ProgramState(uid="u", session_id="s")
    rm = torch.arange(12).view(3, 2, 2).to(torch.int16)
    p.prefix_tree.insert([1, 2, 3], ["a", "b", "c"], [0, 1, 1], [0.0, -1.0, -2.0], rm, step_idx=0)
    (s,) = p.get_steps_from_prefix_tree()
    assert torch.equal(s.moe_routermap, rm) and s.text == "abc"
    st = Step(uid="u", session_id="s")
    st.set_response("ab", [1, 2], [0, 0], [0.0, 0.0], rm[:2])
    st.set_response("c", [3, 4], [1, 1], [-1.0, -1.0], rm[:1])          # shorter: keep head, pad, append
    assert st.moe_routermap.shape == (4, 2, 2) and torch.equal(st.moe_routermap[:2], rm[:2])
    assert bool((st.moe_routermap[2] == -1).all()) and torch.equal(st.moe_routermap[3], rm[0])
    assert not st.is_empty()
    st.mask_out_response()
    assert st.is_empty()


def test_program_manager_group_semantics():
    m = ProgramManager()
    ps = [ProgramState(group_id="g1", uid="a"), ProgramState(group_id="g1", uid="b"), ProgramState(group_id="g2", uid="c")]
    m.add_programs(ps)
    ps[0].done = ps[2].done = True
    assert m.get_num_programs() == 3 and m.get_num_completed_programs() == 2
    got = m.pop_programs(completed=True)
    assert [p.uid for p in got] == ["c"]             # g1 is not fully done
    assert [p.uid for p in m.pop_programs(completed=False)] == ["b"]
    ps[0].done = True
    assert [p.uid for p in m.pop_programs(completed=True)] == ["a"] and m.get_num_programs() == 0
