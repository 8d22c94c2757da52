"""
GSM8K as a generative task with calculator tool calls (reference: tasks/gsm8k.py).

Dataset answers embed `<<expr=result>>` annotations; each becomes a python tool call part
followed by its python_output part, so the model learns to call the calculator.
"""

import re

from tasks.common import Task, load_hub_dataset

_FINAL = re.compile(r"#### (\-?[0-9\.\,]+)")
_CALL = re.compile(r"(<<[^>]+>>)")
GSM_RE = _FINAL                         # name used by code written against the reference


def extract_answer(completion):
    """The number after '####', commas removed; None when absent."""
    m = _FINAL.search(completion)
    return m.group(1).strip().replace(",", "") if m else None


class GSM8K(Task):
    def __init__(self, subset, split, **kwargs):
        super().__init__(**kwargs)
        assert subset in ("main", "socratic"), "GSM8K subset must be main|socratic"
        assert split in ("train", "test"), "GSM8K split must be train|test"
        self.ds = load_hub_dataset("openai/gsm8k", subset, split=split).shuffle(seed=42)

    @property
    def eval_type(self):
        return "generative"

    def num_examples(self):
        return len(self.ds)

    def get_example(self, index):
        row = self.ds[index]
        parts = []
        for piece in _CALL.split(row["answer"]):
            if piece.startswith("<<") and piece.endswith(">>"):
                inner = piece[2:-2]
                expr, result = inner.rsplit("=", 1) if "=" in inner else (inner, "")
                parts.append({"type": "python", "text": expr})
                parts.append({"type": "python_output", "text": result})
            else:
                parts.append({"type": "text", "text": piece})
        return {"messages": [{"role": "user", "content": row["question"]},
                             {"role": "assistant", "content": parts}]}

    def evaluate(self, conversation, assistant_response):
        """1 when the sampled response ends in the same '#### number' as the ground truth."""
        assert isinstance(assistant_response, str), "Assuming simple string response for now"
        truth = conversation["messages"][-1]
        assert truth["role"] == "assistant", "Last message must be from the Assistant"
        assert isinstance(truth["content"], list), "This is expected to be a list of parts"
        want = extract_answer(truth["content"][-1]["text"])
        return int(extract_answer(assistant_response) == want)

    def reward(self, conversation, assistant_response):
        return float(self.evaluate(conversation, assistant_response))
