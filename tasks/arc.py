"""AI2 ARC (Easy / Challenge) as a categorical task (reference: tasks/arc.py)."""

from tasks.common import Task, load_hub_dataset, render_mc


class ARC(Task):
    def __init__(self, subset, split, **kwargs):
        super().__init__(**kwargs)
        assert subset in ("ARC-Easy", "ARC-Challenge"), "ARC subset must be ARC-Easy or ARC-Challenge"
        assert split in ("train", "validation", "test"), "ARC split must be train|validation|test"
        self.ds = load_hub_dataset("allenai/ai2_arc", subset, split=split).shuffle(seed=42)

    @property
    def eval_type(self):
        return "categorical"

    def num_examples(self):
        return len(self.ds)

    def get_example(self, index):
        row = self.ds[index]
        letters = row["choices"]["label"]
        answer = row["answerKey"]
        assert answer in letters, f"ARC answer {answer} must be one of {letters}"
        prompt = render_mc(row["question"], letters, row["choices"]["text"])
        return {"messages": [{"role": "user", "content": prompt}, {"role": "assistant", "content": answer}],
                "letters": letters}

    def evaluate(self, conversation, assistant_response):
        assert assistant_response in conversation["letters"], (
            f"ARC answer {assistant_response} is expected to be one of {conversation['letters']}")
        return assistant_response == conversation["messages"][-1]["content"]
