"""Chat-template rendering and incremental output parsing for the Qwen3.x family.

The template is implemented natively (no Jinja interpreter at run time), as the reference does: a renderer is
selected by the SHA-256 of the artifact's `chat_template.jinja` resource and an unknown template is refused
rather than guessed (src/targets/qwen3_6/impl/frontend/chat_template.cpp:430).  The output side splits the
generated text into reasoning (`<think>` frame), visible content and tool calls (`<tool_call>` JSON frames) while
it streams (src/targets/qwen3_6/impl/frontend/frontend.cpp: thinking / stop / tool-call session).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

IM_START, IM_END = "<|im_start|>", "<|im_end|>"
TOOLS_HEADER = ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                "You are provided with function signatures within <tools></tools> XML tags:\n<tools>")
TOOLS_FOOTER = ("\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
                "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": "
                "<args-json-object>}\n</tool_call>")

# sha256(chat_template.jinja) -> renderer name.  Artifacts written by this package embed the marker template below.
BUILTIN_TEMPLATE = "{# ninfer-fusion-b200 native chat template: qwen3-hybrid-v1 #}\n"
KNOWN_TEMPLATES: Dict[str, str] = {hashlib.sha256(BUILTIN_TEMPLATE.encode()).hexdigest(): "qwen3"}


class TemplateRefused(ValueError):
    pass


def renderer_for(template_text: Optional[str], allow_unknown: bool = False) -> str:
    if template_text is None:
        return "qwen3"
    digest = hashlib.sha256(template_text.encode("utf-8")).hexdigest()
    name = KNOWN_TEMPLATES.get(digest)
    if name is None:
        if allow_unknown:
            return "qwen3"
        raise TemplateRefused(f"chat template {digest[:16]}… is not one of the compiled renderers; refusing to guess")
    return name


def _text_of(content) -> str:
    """OpenAI-style content: a string or a list of typed parts (text parts are concatenated)."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    out = []
    for part in content:
        if isinstance(part, str):
            out.append(part)
        elif part.get("type") in ("text", "input_text", "output_text"):
            out.append(part.get("text", ""))
        elif part.get("type") in ("image_url", "image", "input_image"):
            out.append("<|vision_start|><|image_pad|><|vision_end|>")
        elif part.get("type") in ("video_url", "video"):
            out.append("<|vision_start|><|video_pad|><|vision_end|>")
    return "".join(out)


def render_chat(messages: Sequence[dict], tools: Optional[Sequence[dict]] = None, add_generation_prompt: bool = True,
                enable_thinking: bool = True) -> str:
    """messages: [{"role", "content", optional "reasoning_content", "tool_calls", "tool_call_id"}]."""
    msgs = list(messages)
    out: List[str] = []
    system = ""
    if msgs and msgs[0].get("role") in ("system", "developer"):
        system = _text_of(msgs[0].get("content"))
        msgs = msgs[1:]
    if tools:
        body = (system + "\n\n" if system else "") + TOOLS_HEADER
        for t in tools:
            body += "\n" + json.dumps(t, ensure_ascii=False)
        out.append(f"{IM_START}system\n{body}{TOOLS_FOOTER}{IM_END}\n")
    elif system:
        out.append(f"{IM_START}system\n{system}{IM_END}\n")
    # reasoning of earlier turns is dropped; only turns after the last real user query keep it
    last_query = -1
    for i, m in enumerate(msgs):
        if m.get("role") == "user":
            last_query = i
    i = 0
    while i < len(msgs):
        m = msgs[i]
        role = m.get("role")
        if role in ("user", "system", "developer"):
            out.append(f"{IM_START}{'system' if role != 'user' else 'user'}\n{_text_of(m.get('content'))}{IM_END}\n")
        elif role == "assistant":
            content = _text_of(m.get("content"))
            reasoning = m.get("reasoning_content") or ""
            if not reasoning and "</think>" in content:
                head, _, content = content.partition("</think>")
                reasoning = head.split("<think>")[-1].strip("\n")
                content = content.lstrip("\n")
            block = f"{IM_START}assistant\n"
            if reasoning and i > last_query:
                block += f"<think>\n{reasoning.strip()}\n</think>\n\n"
            block += content
            for k, call in enumerate(m.get("tool_calls") or []):
                fn = call.get("function", call)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except json.JSONDecodeError:
                        pass
                if content or k > 0:
                    block += "\n"
                block += "<tool_call>\n" + json.dumps({"name": fn.get("name"), "arguments": args}, ensure_ascii=False) + "\n</tool_call>"
            out.append(block + f"{IM_END}\n")
        elif role == "tool":
            # consecutive tool results share one user frame
            block = f"{IM_START}user"
            while i < len(msgs) and msgs[i].get("role") == "tool":
                block += f"\n<tool_response>\n{_text_of(msgs[i].get('content'))}\n</tool_response>"
                i += 1
            out.append(block + f"{IM_END}\n")
            continue
        else:
            raise ValueError(f"unknown message role '{role}'")
        i += 1
    if add_generation_prompt:
        out.append(f"{IM_START}assistant\n")
        if not enable_thinking:
            out.append("<think>\n\n</think>\n\n")
    return "".join(out)


# ---------------------------------------------------------------------------------------------------------
# Incremental output parsing
# ---------------------------------------------------------------------------------------------------------
@dataclass
class ToolCall:
    name: str
    arguments: str        # JSON text of the arguments object
    raw: str = ""


@dataclass
class ParsedDelta:
    reasoning: str = ""
    content: str = ""
    tool_calls: List[ToolCall] = field(default_factory=list)


class OutputParser:
    """Feeds on decoded text fragments and separates reasoning / content / tool calls as they stream.

    `thinking=True` means the generation prompt left the model inside an open reasoning frame (the Qwen3 prompt
    does not emit `<think>` itself when thinking is enabled by default in newer templates; an explicit `<think>`
    at the start is accepted too).  Text that could be the beginning of a tag is held back until it is
    disambiguated, so a client never sees half a tag."""

    TAGS = ("<think>", "</think>", "<tool_call>", "</tool_call>")

    def __init__(self, thinking: bool = False, stop: Sequence[str] = ()):
        self.mode = "reasoning" if thinking else "content"
        self.stop = [s for s in stop if s]
        self.stopped = False
        self._hold = ""
        self._tool = ""
        self.reasoning = ""
        self.content = ""
        self.tool_calls: List[ToolCall] = []

    def _emit(self, delta: ParsedDelta, text: str) -> None:
        if not text:
            return
        if self.mode == "reasoning":
            delta.reasoning += text
            self.reasoning += text
        elif self.mode == "tool":
            self._tool += text
        else:
            delta.content += text
            self.content += text

    def _close_tool(self, delta: ParsedDelta) -> None:
        raw = self._tool.strip()
        self._tool = ""
        try:
            obj = json.loads(raw)
            args = obj.get("arguments", {})
            call = ToolCall(str(obj.get("name", "")), args if isinstance(args, str) else json.dumps(args, ensure_ascii=False), raw)
        except (json.JSONDecodeError, AttributeError):
            call = ToolCall("", raw, raw)   # malformed: surfaced verbatim, the gateway decides what to do with it
        delta.tool_calls.append(call)
        self.tool_calls.append(call)

    def feed(self, text: str) -> ParsedDelta:
        delta = ParsedDelta()
        if self.stopped:
            return delta
        buf = self._hold + text
        self._hold = ""
        markers = list(self.TAGS) + (self.stop if self.mode == "content" else [])
        while buf:
            # earliest complete marker
            pos, hit = -1, None
            for m in markers:
                p = buf.find(m)
                if p >= 0 and (pos < 0 or p < pos or (p == pos and len(m) > len(hit))):
                    pos, hit = p, m
            if hit is None:
                # hold back a suffix that is a proper prefix of some marker
                keep = 0
                for m in markers:
                    for n in range(min(len(m) - 1, len(buf)), 0, -1):
                        if buf.endswith(m[:n]):
                            keep = max(keep, n)
                            break
                self._emit(delta, buf[:len(buf) - keep])
                self._hold = buf[len(buf) - keep:]
                break
            self._emit(delta, buf[:pos])
            buf = buf[pos + len(hit):]
            if hit in self.stop and self.mode == "content":
                self.stopped = True
                break
            if hit == "<think>":
                self.mode = "reasoning"
            elif hit == "</think>":
                self.mode = "content"
                buf = buf.lstrip("\n") if buf else buf
                if not buf:
                    self._strip_newlines = True
            elif hit == "<tool_call>":
                self.mode = "tool"
            elif hit == "</tool_call>":
                self._close_tool(delta)
                self.mode = "content"
            markers = list(self.TAGS) + (self.stop if self.mode == "content" else [])
        if getattr(self, "_strip_newlines", False) and delta.content:
            stripped = delta.content.lstrip("\n")
            self.content = self.content[: len(self.content) - len(delta.content)] + stripped
            delta.content = stripped
            if stripped:
                self._strip_newlines = False
        return delta

    def finish(self) -> ParsedDelta:
        """End of generation: flush held-back text (an unterminated tool frame is surfaced as content)."""
        delta = ParsedDelta()
        if self.stopped:
            return delta
        tail, self._hold = self._hold, ""
        if self.mode == "tool":
            self.mode = "content"
            tail = "<tool_call>" + self._tool + tail
            self._tool = ""
        self._emit(delta, tail)
        return delta
