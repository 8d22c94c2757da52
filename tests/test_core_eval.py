"""
CPU tests of the CORE evaluation: prompt layouts, common prefix / suffix spans, and the three scoring rules with a
toy model whose preferences are known (it always predicts "previous token + 1").
"""
import torch

from nanochat_b200 import core_eval as ce


class _CharTok:
    """One token per character (codes 1..255), BOS = 0."""

    def get_bos_token_id(self):
        return 0

    def __call__(self, prompts, prepend=None):
        out = []
        for p in prompts:
            ids = [min(ord(c), 255) for c in p]
            out.append(([prepend] if prepend is not None else []) + ids)
        return out


class _SuccessorModel:
    """Logits that put almost all mass on (previous token + 1) mod 256."""

    def __call__(self, ids):
        B, T = ids.shape
        logits = torch.full((B, T, 256), -10.0)
        logits.scatter_(2, ((ids + 1) % 256).unsqueeze(-1), 10.0)
        return logits


def test_prompt_layouts():
    shots = [{"query": "Q1", "choices": ["a", "b"], "gold": 1}]
    item = {"query": "Q2", "choices": ["x", "y", "z"], "gold": 0}
    assert ce.render_prompts_mc(item, " -> ", shots) == ["Q1 -> b\n\nQ2 -> x", "Q1 -> b\n\nQ2 -> y", "Q1 -> b\n\nQ2 -> z"]
    schema = {"context_options": ["c1", "c2"], "continuation": "end", "gold": 1}
    assert ce.render_prompts_schema(schema, " ", None) == ["c1 end", "c2 end"]
    lm = {"context": "  the cat ", "continuation": "sat"}
    without, with_c = ce.render_prompts_lm(lm, " ", None)
    assert without == "the cat" and with_c == "the cat sat" and with_c.startswith(without)


def test_common_prefix_and_suffix_lengths():
    seqs = [[1, 2, 3, 9, 7, 7], [1, 2, 3, 4, 5, 7, 7], [1, 2, 3, 7, 7]]
    assert ce.find_common_length(seqs, "left") == 3
    assert ce.find_common_length(seqs, "right") == 2
    tok = _CharTok()
    tokens, starts, ends = ce.batch_sequences_mc(tok, ["ab: x", "ab: yy"])
    assert starts == [5, 5] and ends == [6, 7]                     # BOS + "ab: " is shared
    tokens, starts, ends = ce.batch_sequences_schema(tok, ["p end", "qq end"])
    assert [e - s for s, e in zip(starts, ends)] == [4, 4]         # " end" is the shared continuation
    padded = ce.stack_sequences(tokens, 0)
    assert padded.shape == (2, 7) and padded[0, -1].item() == 0


def test_scoring_rules_with_a_model_of_known_preferences():
    tok, model = _CharTok(), _SuccessorModel()
    meta = {"task_type": "multiple_choice", "num_fewshot": 0, "continuation_delimiter": ""}
    # after "abc" the successor model wants "d": choice 1 is the likely continuation
    data = [{"query": "abc", "choices": ["x", "d", "q"], "gold": 1}, {"query": "abc", "choices": ["x", "d", "q"], "gold": 0}]
    assert ce.evaluate_example(0, model, tok, data, "cpu", meta) is True
    assert ce.evaluate_example(1, model, tok, data, "cpu", meta) is False
    # schema: the continuation "d" is likely after context "abc", unlikely after "abz"
    meta = {"task_type": "schema", "num_fewshot": 0, "continuation_delimiter": ""}
    data = [{"context_options": ["abz", "abc"], "continuation": "d", "gold": 1}]
    assert ce.evaluate_example(0, model, tok, data, "cpu", meta) is True
    # language modelling: every continuation token must be the argmax
    meta = {"task_type": "language_modeling", "num_fewshot": 0, "continuation_delimiter": ""}
    data = [{"context": "abc", "continuation": "def"}, {"context": "abc", "continuation": "dxf"}]
    assert ce.evaluate_example(0, model, tok, data, "cpu", meta) is True
    assert ce.evaluate_example(1, model, tok, data, "cpu", meta) is False
    # few-shot examples come from the other items, deterministically per index
    meta = {"task_type": "multiple_choice", "num_fewshot": 1, "continuation_delimiter": ""}
    data = [{"query": "abc", "choices": ["x", "d"], "gold": 1}, {"query": "klm", "choices": ["n", "z"], "gold": 0}]
    assert ce.evaluate_example(0, model, tok, data, "cpu", meta) is True
    acc = ce.evaluate_task(model, tok, data, "cpu", meta)
    assert acc == 1.0
