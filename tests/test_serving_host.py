"""Host side of the chat front ends without a GPU: message normalisation, tool-call and thinking parsing, the
incremental detokeniser, the reply objects and the HTTP framing, driven by a scripted session."""

import json
import threading
import urllib.request

from megakernels_b200 import server
from megakernels_b200.chat import TextStream, repl


class ByteTokenizer:
    """ids are UTF-8 bytes; 256 is the stop id."""

    def encode(self, text):
        return list(text.encode())

    def decode(self, ids):
        return bytes(i for i in ids if i < 256).decode(errors="replace")


class ScriptedSession:
    """Answers every prompt with a fixed text, then the stop id."""

    def __init__(self, reply):
        self.tok, self.stop_ids, self.reply, self.stats, self.prompts = ByteTokenizer(), [256], reply, {}, []

    def render(self, messages, enable_thinking=False, tools=None):
        return "".join(f"<{m['role']}>{m['content']}" for m in messages) + "<assistant>"

    def encode(self, text):
        return self.tok.encode(text)

    def stream(self, prompt, max_new_tokens=512, temperature=0.7, seed=None):
        self.prompts.append(bytes(prompt).decode())
        ids = self.tok.encode(self.reply)[:max_new_tokens]
        yield from ids
        if len(ids) < max_new_tokens:
            yield 256
        self.stats = dict(prefill_tokens=len(prompt), prefill_s=0.0, decode_tokens=len(ids), decode_s=1.0, decode_tok_s=float(len(ids)))

    def chat(self, messages, enable_thinking=False, tools=None, **kw):
        for t in self.stream(self.encode(self.render(messages)), **kw):
            if t not in self.stop_ids:
                yield t


def test_messages_are_normalised():
    got = server.plain_messages([
        {"role": "user", "content": [{"type": "text", "text": "a"}, {"type": "image_url", "image_url": "x"}, {"text": "b"}]},
        {"role": "assistant", "content": None, "tool_calls": [{"function": {"name": "f", "arguments": "{\"x\": 1}"}},
                                                            {"function": {"name": "g", "arguments": "not json"}}]}])
    assert got[0]["content"] == "ab" and got[1]["content"] == ""
    assert got[1]["tool_calls"][0]["function"]["arguments"] == {"x": 1}
    assert got[1]["tool_calls"][1]["function"]["arguments"] == {"input": "not json"}


def test_tool_calls_and_thinking_are_parsed():
    text = "<think>plan</think>\nSure.<tool_call>\n<function=get_weather>\n<parameter=city>\n\"Oslo\"\n</parameter>\n<parameter=unit>\nC\n</parameter>\n</function>\n</tool_call>"
    answer, thought = server.split_thinking(text)
    assert thought == "plan" and answer.startswith("Sure.")
    content, calls = server.extract_tool_calls(answer)
    assert content == "Sure." and len(calls) == 1 and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo", "unit": "C"}
    assert server.extract_tool_calls("no calls") == ("no calls", []) and server.split_thinking("x") == ("x", None)


def test_text_stream_holds_back_half_characters():
    ts = TextStream(ByteTokenizer())
    pieces = [ts.push(b) for b in "aé€".encode()]
    assert pieces == ["a", "", "é", "", "", "€"] and "".join(pieces) == "aé€"


def test_completion_object():
    s = ScriptedSession("<think>t</think>hello")
    r = server.complete(s, {"messages": [{"role": "user", "content": "hi"}], "enable_thinking": True, "max_tokens": 64})
    c = r["choices"][0]
    assert c["finish_reason"] == "stop" and c["message"] == {"role": "assistant", "content": "hello", "reasoning_content": "t"}
    assert r["usage"]["completion_tokens"] == len("<think>t</think>hello") + 1 and r["object"] == "chat.completion"
    r = server.complete(s, {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
    assert r["choices"][0]["finish_reason"] == "length"


def test_streamed_chunks_carry_reasoning_answer_and_tool_calls():
    reply = "<think>why</think>\n\nOK <tool_call>\n<function=f>\n<parameter=a>\n1\n</parameter>\n</function>\n</tool_call>"
    s = ScriptedSession(reply)
    req = {"messages": [{"role": "user", "content": "x"}], "stream": True, "tools": [{"type": "function"}],
           "chat_template_kwargs": {"enable_thinking": True}}
    chunks = list(server.stream_chunks(s, req))
    deltas = [c["choices"][0]["delta"] for c in chunks]
    assert deltas[0] == {"role": "assistant", "content": ""}
    assert "".join(d.get("reasoning_content", "") for d in deltas) == "why"
    assert "".join(d.get("content", "") for d in deltas) == "OK "
    calls = [d["tool_calls"] for d in deltas if "tool_calls" in d]
    assert len(calls) == 1 and calls[0][0]["function"]["name"] == "f" and calls[0][0]["index"] == 0
    assert chunks[-1]["choices"][0]["finish_reason"] == "tool_calls" and len({c["id"] for c in chunks}) == 1


def test_http_round_trip():
    s = ScriptedSession("pong")
    httpd = server.serve(s, "127.0.0.1", 0)
    port = httpd.server_address[1]
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    try:
        base = f"http://127.0.0.1:{port}"
        assert json.load(urllib.request.urlopen(base + "/v1/models"))["data"][0]["id"] == server.MODEL_ID
        assert json.load(urllib.request.urlopen(base + "/health")) == {"status": "ok"}
        body = json.dumps({"messages": [{"role": "user", "content": "ping"}]}).encode()
        r = json.load(urllib.request.urlopen(urllib.request.Request(base + "/v1/chat/completions", data=body)))
        assert r["choices"][0]["message"]["content"] == "pong" and s.prompts[-1] == "<user>ping<assistant>"
        body = json.dumps({"messages": [{"role": "user", "content": "ping"}], "stream": True}).encode()
        raw = urllib.request.urlopen(urllib.request.Request(base + "/v1/chat/completions", data=body)).read().decode()
        events = [json.loads(x[len("data: "):]) for x in raw.split("\n\n") if x.startswith("data: {")]
        assert "".join(e["choices"][0]["delta"].get("content", "") for e in events) == "pong" and raw.rstrip().endswith("data: [DONE]")
        try:
            urllib.request.urlopen(urllib.request.Request(base + "/v1/chat/completions", data=b"{}"))
            assert False, "a request without messages must be refused"
        except urllib.error.HTTPError as e:
            assert e.code == 400
    finally:
        httpd.shutdown()


def test_repl_commands():
    s = ScriptedSession("hi there")
    lines = iter(["hello", "/stats", "/reset", "again", "/quit"])
    out = []

    class Out:
        def write(self, t):
            out.append(t)

        def flush(self):
            pass

    repl(s, system="be brief", inp=lambda prompt: next(lines), out=Out())
    text = "".join(out)
    assert text.count("hi there") == 2 and "(conversation cleared)" in text and "tok/s" in text
    assert s.prompts[0] == "<system>be brief<user>hello<assistant>" and s.prompts[1] == "<system>be brief<user>again<assistant>"
