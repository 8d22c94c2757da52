"""
Talk to a finetuned model from the terminal (single GPU or CPU).

    python -m scripts.chat_cli                 # interactive; 'clear' restarts, 'quit' exits
    python -m scripts.chat_cli -p "Why is the sky blue?"

The conversation is kept as one token stream: <|bos|> then, per turn,
<|user_start|> text <|user_end|> <|assistant_start|> reply <|assistant_end|>; replies are
streamed token by token from `Engine.generate` (reference: scripts/chat_cli.py).
"""
import argparse

from nanochat_b200.common import compute_init, autodetect_device_type
from nanochat_b200.engine import Engine
from nanochat_b200.checkpoint_manager import load_model


def main():
    ap = argparse.ArgumentParser(description="Chat with the model")
    ap.add_argument("-i", "--source", type=str, default="sft", help="sft|rl|base")
    ap.add_argument("-g", "--model-tag", type=str, default=None)
    ap.add_argument("-s", "--step", type=int, default=None)
    ap.add_argument("-p", "--prompt", type=str, default="", help="ask once and exit")
    ap.add_argument("-t", "--temperature", type=float, default=0.6)
    ap.add_argument("-k", "--top-k", type=int, default=50)
    ap.add_argument("--device-type", type=str, default="", choices=["cuda", "cpu", "mps", ""])
    args = ap.parse_args()

    device_type = autodetect_device_type() if args.device_type == "" else args.device_type
    _, _, _, _, device = compute_init(device_type)
    model, tokenizer, _ = load_model(args.source, device, phase="eval", model_tag=args.model_tag, step=args.step)
    engine = Engine(model, tokenizer)
    sp = tokenizer.encode_special
    bos, assistant_end = tokenizer.get_bos_token_id(), sp("<|assistant_end|>")

    print("\nNanoChat Interactive Mode\n" + "-" * 50)
    print("Type 'quit' or 'exit' to end the conversation\nType 'clear' to start a new conversation\n" + "-" * 50)
    history = [bos]
    while True:
        if args.prompt:
            text = args.prompt
        else:
            try:
                text = input("\nUser: ").strip()
            except (EOFError, KeyboardInterrupt):
                print("\nGoodbye!")
                break
        if text.lower() in ("quit", "exit"):
            print("Goodbye!")
            break
        if text.lower() == "clear":
            history = [bos]
            print("Conversation cleared.")
            continue
        if not text:
            continue
        history += [sp("<|user_start|>"), *tokenizer.encode(text), sp("<|user_end|>"), sp("<|assistant_start|>")]
        reply = []
        print("\nAssistant: ", end="", flush=True)
        for column, _ in engine.generate(history, num_samples=1, max_tokens=256, temperature=args.temperature,
                                         top_k=args.top_k):
            reply.append(column[0])
            print(tokenizer.decode([column[0]]), end="", flush=True)
        print()
        if not reply or reply[-1] != assistant_end:
            reply.append(assistant_end)     # generation stopped on the token budget: close the turn ourselves
        history += reply
        if args.prompt:
            break


if __name__ == "__main__":
    main()
