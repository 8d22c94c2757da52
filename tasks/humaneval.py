"""HumanEval as a generative task scored by running the tests in the sandbox (reference: tasks/humaneval.py)."""

import re

from nanochat_b200.execution import execute_code
from tasks.common import Task, load_hub_dataset


def extract_imports(prompt):
    """Leading import lines of a code prompt."""
    found = []
    for line in prompt.split("\n"):
        s = line.strip()
        if s.startswith("import ") or s.startswith("from "):
            found.append(s)
        elif s and not s.startswith("#"):
            break
    return "\n".join(found)


def extract_program(completion):
    """First fenced code block of a completion, else the whole text."""
    blocks = re.findall(r"```(?:python)?\s*\n(.*?)\n```", completion, re.DOTALL)
    return (blocks[0] if blocks else completion).strip()


class HumanEval(Task):
    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.ds = load_hub_dataset("openai/openai_humaneval", subset="openai_humaneval", split="test").shuffle(seed=42)

    @property
    def eval_type(self):
        return "generative"

    def num_examples(self):
        return len(self.ds)

    def get_example(self, index):
        row = self.ds[index]
        prompt = row["prompt"]
        return {"messages": [{"role": "user", "content": prompt},
                             {"role": "assistant", "content": f"{prompt}\n{row['canonical_solution']}"}],
                "entry_point": row["entry_point"], "test": row["test"]}

    def evaluate(self, conversation, completion):
        program = "\n\n".join([extract_imports(conversation["messages"][0]["content"]),
                               extract_program(completion), conversation["test"]])
        program += f"\ncheck({conversation['entry_point']})"
        return execute_code(program).success
