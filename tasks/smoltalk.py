"""smol-smoltalk conversations for SFT (reference: tasks/smoltalk.py). train ~460K rows, test ~24K."""

from tasks.common import Task, load_hub_dataset


class SmolTalk(Task):
    def __init__(self, split, **kwargs):
        super().__init__(**kwargs)
        assert split in ("train", "test"), "SmolTalk split must be train|test"
        self.ds = load_hub_dataset("HuggingFaceTB/smol-smoltalk", split=split).shuffle(seed=42)
        self.length = len(self.ds)

    def num_examples(self):
        return self.length

    def get_example(self, index):
        messages = self.ds[index]["messages"]
        assert len(messages) >= 1
        turns = messages[1:] if messages[0]["role"] == "system" else messages
        assert len(turns) >= 2, "SmolTalk messages must have at least 2 messages"
        for i, m in enumerate(turns):
            want = "user" if i % 2 == 0 else "assistant"
            assert m["role"] == want, f"Message {i} has role {m['role']} but should be {want}"
            assert isinstance(m["content"], str), "Content must be a string"
        return {"messages": messages}
