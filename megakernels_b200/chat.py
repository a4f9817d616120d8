"""Interactive chat on the 0.8B engine, and the incremental detokeniser the server shares.

    python -m megakernels_b200.chat --model /path/to/snapshot [--temperature 0.7] [--system "..."] [--think]

Commands: /reset clears the conversation, /stats toggles the speed line, /quit exits.  The counterpart of the
reference's `qwen-mk-chat` (`qwen3.5-0.8b/qwen_mk/chat.py:14-86`)."""

import argparse
import sys


class TextStream:
    """Turns a stream of ids into a stream of text, holding back output while it ends inside a multi-byte character."""

    def __init__(self, tokenizer):
        self.tok, self.ids, self.shown = tokenizer, [], 0

    def push(self, token):
        self.ids.append(token)
        text = self.tok.decode(self.ids)
        if text.endswith("�"):
            return ""
        fresh, self.shown = text[self.shown:], len(text)
        return fresh


def repl(session, system=None, temperature=0.7, max_new_tokens=2048, think=False, inp=input, out=sys.stdout):
    """The read-reply loop.  `inp` / `out` are injectable for tests."""
    base = [{"role": "system", "content": system}] if system else []
    messages, show_stats = list(base), True
    while True:
        try:
            line = inp("\n> ")
        except (EOFError, KeyboardInterrupt):
            return
        word = line.strip()
        if word in ("/quit", "/exit"):
            return
        if word == "/reset":
            messages = list(base)
            out.write("(conversation cleared)\n")
            continue
        if word == "/stats":
            show_stats = not show_stats
            continue
        if not word:
            continue
        messages.append({"role": "user", "content": line})
        text, stream = "", TextStream(session.tok)
        for t in session.chat(messages, enable_thinking=think, temperature=temperature, max_new_tokens=max_new_tokens):
            piece = stream.push(t)
            text += piece
            out.write(piece)
            out.flush()
        out.write("\n")
        messages.append({"role": "assistant", "content": text.split("</think>")[-1].strip()})
        if show_stats and session.stats:
            s = session.stats
            out.write(f"[{s['decode_tokens']} tokens, {s['decode_tok_s']:.0f} tok/s; prompt: {s['prefill_tokens']} new tokens in {s['prefill_s']:.2f} s]\n")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="local snapshot directory (this library never downloads)")
    ap.add_argument("--temperature", type=float, default=0.7, help="0 = greedy")
    ap.add_argument("--max-new-tokens", type=int, default=2048)
    ap.add_argument("--system", default=None)
    ap.add_argument("--think", action="store_true")
    ap.add_argument("--max-seq", type=int, default=32768)
    ap.add_argument("--quant", choices=["int8", "bf16"], default="int8")
    ap.add_argument("--no-spec", action="store_true", help="one token per step instead of speculative cycles (same output)")
    args = ap.parse_args()
    from .session import ChatSession
    session = ChatSession.from_snapshot(args.model, max_seq=args.max_seq, quant=args.quant, spec=not args.no_spec)
    print("ready. /reset, /stats, /quit", file=sys.stderr)
    repl(session, args.system, args.temperature, args.max_new_tokens, args.think)


if __name__ == "__main__":
    main()
