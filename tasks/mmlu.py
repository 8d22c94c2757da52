"""MMLU as a categorical task (reference: tasks/mmlu.py)."""

from tasks.common import Task, load_hub_dataset, render_mc


class MMLU(Task):
    letters = ("A", "B", "C", "D")

    def __init__(self, subset, split, **kwargs):
        super().__init__(**kwargs)
        assert subset in ("all",), f"subset {subset} must be all"
        assert split in ("auxiliary_train", "validation", "dev", "test"), (
            f"split {split} must be auxiliary_train|validation|dev|test")
        self.subset, self.split = subset, split
        self.ds = load_hub_dataset("cais/mmlu", subset, split=split).shuffle(seed=42)

    @property
    def eval_type(self):
        return "categorical"

    def num_examples(self):
        return len(self.ds)

    def get_example(self, index):
        row = self.ds[index]
        choices = row["choices"]
        assert len(choices) == 4, "MMLU should have 4 choices"
        prompt = render_mc(row["question"], self.letters, choices)
        return {"messages": [{"role": "user", "content": prompt},
                             {"role": "assistant", "content": self.letters[row["answer"]]}],
                "subject": row["subject"], "letters": self.letters}

    def evaluate(self, conversation, assistant_response):
        assert assistant_response in self.letters, (
            f"MMLU answer {assistant_response} is expected to be one of {self.letters}")
        return assistant_response == conversation["messages"][-1]["content"]
