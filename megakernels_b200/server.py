"""OpenAI-compatible HTTP front end of a `ChatSession` (standard library only).

    python -m megakernels_b200.server --model /path/to/snapshot --port 8000
    curl localhost:8000/v1/chat/completions -d '{"messages":[{"role":"user","content":"hi"}]}'

Endpoints and request fields of the reference's server (`qwen3.5-0.8b/qwen_mk/server.py:27-209`): GET /v1/models and
/health; POST /v1/chat/completions with `messages`, `stream`, `max_tokens` / `max_completion_tokens`, `temperature`,
`seed`, `tools`, `enable_thinking` (also under `chat_template_kwargs`).  Replies carry `reasoning_content` for a
`<think>` block and `tool_calls` parsed from the model's XML tool-call format.  One engine, one sequence: requests
are served one at a time (the session's lock), and consecutive requests of a conversation reuse the state.
"""

import argparse
import json
import re
import sys
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .chat import TextStream

MODEL_ID = "qwen3.5-0.8b-megakernel-b200"
_CALL = re.compile(r"<tool_call>\s*<function=([^>\s]+)>(.*?)</function>\s*</tool_call>", re.S)
_PARAM = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


def plain_messages(messages):
    """OpenAI message objects -> what a chat template takes: text content, tool-call arguments as objects."""
    result = []
    for msg in messages:
        msg = dict(msg)
        content = msg.get("content")
        if isinstance(content, list):
            content = "".join(part.get("text", "") for part in content if part.get("type") in (None, "text"))
        msg["content"] = content or ""
        if msg.get("tool_calls"):
            fixed = []
            for call in msg["tool_calls"]:
                fn = dict(call.get("function", call))
                if isinstance(fn.get("arguments"), str):
                    try:
                        fn["arguments"] = json.loads(fn["arguments"] or "{}")
                    except json.JSONDecodeError:
                        fn["arguments"] = {"input": fn["arguments"]}
                fixed.append({"type": "function", "function": fn})
            msg["tool_calls"] = fixed
        result.append(msg)
    return result


def extract_tool_calls(text):
    """(text without the tool-call blocks, OpenAI tool_calls list)."""
    calls = []
    for name, body in _CALL.findall(text):
        args = {}
        for key, raw in _PARAM.findall(body):
            try:
                args[key] = json.loads(raw)
            except json.JSONDecodeError:
                args[key] = raw
        calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                      "function": {"name": name, "arguments": json.dumps(args)}})
    return (_CALL.sub("", text).strip() if calls else text), calls


def split_thinking(text):
    """(answer, reasoning or None)."""
    if "</think>" not in text:
        return text, None
    thought, _, answer = text.partition("</think>")
    return answer.strip(), thought.replace("<think>", "").strip()


def settled(text, tag):
    """`text` without a trailing fragment that may still grow into `tag` (tags can arrive a character at a time)."""
    for n in range(min(len(tag) - 1, len(text)), 0, -1):
        if text.endswith(tag[:n]):
            return text[:-n]
    return text


def complete(session, req):
    """The non-streaming reply object for a parsed request body."""
    messages = plain_messages(req["messages"])
    think = bool(req.get("enable_thinking", (req.get("chat_template_kwargs") or {}).get("enable_thinking", False)))
    tools = req.get("tools") or None
    prompt = session.encode(session.render(messages, enable_thinking=think, tools=tools))
    budget = int(req.get("max_completion_tokens") or req.get("max_tokens") or 2048)
    ids = list(session.stream(prompt, max_new_tokens=budget, temperature=float(req.get("temperature", 0.7)), seed=req.get("seed")))
    finish = "stop" if ids and ids[-1] in session.stop_ids else "length"
    text, reasoning = split_thinking(session.tok.decode([t for t in ids if t not in session.stop_ids]))
    content, calls = extract_tool_calls(text)
    message = {"role": "assistant", "content": content or (None if calls else "")}
    if calls:
        message["tool_calls"], finish = calls, "tool_calls"
    if reasoning is not None:
        message["reasoning_content"] = reasoning
    return {"id": "chatcmpl-" + uuid.uuid4().hex, "object": "chat.completion", "created": int(time.time()), "model": MODEL_ID,
            "choices": [{"index": 0, "message": message, "finish_reason": finish}],
            "usage": {"prompt_tokens": len(prompt), "completion_tokens": len(ids), "total_tokens": len(prompt) + len(ids)}}


def stream_chunks(session, req):
    """Generator of chat.completion.chunk objects for a streaming request (the caller frames them as SSE)."""
    messages = plain_messages(req["messages"])
    think = bool(req.get("enable_thinking", (req.get("chat_template_kwargs") or {}).get("enable_thinking", False)))
    tools = req.get("tools") or None
    prompt = session.encode(session.render(messages, enable_thinking=think, tools=tools))
    budget = int(req.get("max_completion_tokens") or req.get("max_tokens") or 2048)
    cid, created = "chatcmpl-" + uuid.uuid4().hex, int(time.time())

    def chunk(delta, finish=None):
        return {"id": cid, "object": "chat.completion.chunk", "created": created, "model": MODEL_ID,
                "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}

    yield chunk({"role": "assistant", "content": ""})
    pieces, text = TextStream(session.tok), ""
    sent_thought = sent_answer = 0
    answer_from = None if think else 0          # index in `text` where the visible answer begins
    finish = "length"
    for t in session.stream(prompt, max_new_tokens=budget, temperature=float(req.get("temperature", 0.7)), seed=req.get("seed")):
        if t in session.stop_ids:               # always the last id; keep iterating so the session closes its ledger
            finish = "stop"
            continue
        text += pieces.push(t)
        if answer_from is None:
            opening = text.lstrip()
            if len(opening) < len("<think>") and "<think>".startswith(opening):
                continue                                    # the opening tag is still arriving
            thought = settled(text.split("</think>")[0], "</think>").replace("<think>", "")
            if len(thought) > sent_thought:
                yield chunk({"reasoning_content": thought[sent_thought:]})
                sent_thought = len(thought)
            if "</think>" in text:
                answer_from = text.index("</think>") + len("</think>")
            continue
        answer = text[answer_from:]
        if sent_answer == 0:
            stripped = answer.lstrip("\n")
            answer_from += len(answer) - len(stripped)
            answer = stripped
        visible = settled(answer.split("<tool_call>")[0], "<tool_call>") if tools else answer
        if len(visible) > sent_answer:
            yield chunk({"content": visible[sent_answer:]})
            sent_answer = len(visible)
    if answer_from is not None and tools:
        content, calls = extract_tool_calls(text[answer_from:])
        if calls:
            yield chunk({"tool_calls": [dict(c, index=i) for i, c in enumerate(calls)]})
            finish = "tool_calls"
        elif len(content) > sent_answer:
            yield chunk({"content": content[sent_answer:]})
    yield chunk({}, finish)


class Handler(BaseHTTPRequestHandler):
    session = None
    protocol_version = "HTTP/1.1"

    def log_message(self, fmt, *args):
        sys.stderr.write("[mk-b200] " + fmt % args + "\n")

    def _reply(self, code, obj):
        body = json.dumps(obj).encode()
        self.send_response(code)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def do_GET(self):
        path = self.path.rstrip("/")
        if path in ("/v1/models", "/models"):
            self._reply(200, {"object": "list", "data": [{"id": MODEL_ID, "object": "model", "owned_by": "local"}]})
        elif path in ("", "/health"):
            self._reply(200, {"status": "ok"})
        else:
            self._reply(404, {"error": {"message": "not found"}})

    def do_POST(self):
        if self.path.rstrip("/") not in ("/v1/chat/completions", "/chat/completions"):
            return self._reply(404, {"error": {"message": "not found"}})
        try:
            req = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
            if not isinstance(req.get("messages"), list):
                raise KeyError("messages")
        except (ValueError, KeyError) as e:
            return self._reply(400, {"error": {"message": f"bad request: {e}"}})
        if not req.get("stream"):
            return self._reply(200, complete(self.session, req))
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.send_header("Cache-Control", "no-cache")
        self.send_header("Transfer-Encoding", "chunked")
        self.end_headers()

        def frame(payload):
            self.wfile.write(f"{len(payload):x}\r\n".encode() + payload + b"\r\n")
            self.wfile.flush()

        chunks = stream_chunks(self.session, req)
        try:
            for c in chunks:
                frame(f"data: {json.dumps(c)}\n\n".encode())
            frame(b"data: [DONE]\n\n")
            self.wfile.write(b"0\r\n\r\n")
            self.wfile.flush()
        except (BrokenPipeError, ConnectionResetError):
            chunks.close()


def serve(session, host="127.0.0.1", port=8000):
    Handler.session = session
    return ThreadingHTTPServer((host, port), Handler)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="local snapshot directory (this library never downloads)")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max-seq", type=int, default=32768)
    ap.add_argument("--quant", choices=["int8", "bf16"], default="int8")
    ap.add_argument("--no-spec", action="store_true")
    args = ap.parse_args()
    from .session import ChatSession
    session = ChatSession.from_snapshot(args.model, max_seq=args.max_seq, quant=args.quant, spec=not args.no_spec)
    httpd = serve(session, args.host, args.port)
    print(f"serving {MODEL_ID} on http://{args.host}:{args.port}/v1", file=sys.stderr)
    httpd.serve_forever()


if __name__ == "__main__":
    main()
