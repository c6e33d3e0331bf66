"""Chat templates of widely used model families rendered by the router's template bridge and compared with
the expected prompts.  The vectors (template text, conversation, expected output) are the cases of the
reference's template test (`router/src/infer/chat_template.rs:739-1168`), kept as data in
`tests/data/chat_templates.json`; the remaining cases cover `raise_exception`, loop controls, `strftime_now`,
generation-prompt handling and tool descriptions."""
import datetime
import json
import os

import pytest

from tgi_b200.router import pybridge

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = json.load(open(os.path.join(HERE, "data", "chat_templates.json")))
CHAT = [{"role": "user", "content": "Hello, how are you?"},
        {"role": "assistant", "content": "I'm doing great. How can I help you today?"},
        {"role": "user", "content": "I'd like to show off how chat templating works!"}]
SYSTEM = [{"role": "system", "content": "You are a friendly chatbot who always responds in the style of a pirate"}]


def render(template, messages, add_generation_prompt=False, bos="", eos="", **extra):
    pybridge._STATE.update(chat_template=template, bos_token=bos, eos_token=eos)
    out = json.loads(pybridge.apply_chat_template(json.dumps(
        dict(messages=messages, add_generation_prompt=add_generation_prompt, **extra))))
    return out


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_model_family_templates(case):
    messages = case["messages"] if isinstance(case["messages"], list) else \
        ((SYSTEM + CHAT) if case["messages"] == "system" else CHAT)
    out = render(case["chat_template"], messages, case["add_generation_prompt"], case["bos_token"] or "",
                 case["eos_token"] or "")
    assert out.get("ok"), out
    assert out["text"] == case["target"]


def test_raise_exception_surfaces_as_a_template_error():
    tpl = ("{{ bos_token }}{% for message in messages %}{% if (message['role'] == 'user') != (loop.index0 % 2 == 0) %}"
           "{{ raise_exception('Conversation roles must alternate user/assistant/user/assistant/...') }}{% endif %}"
           "{{ message['content'] }}{% endfor %}")
    bad = [{"role": "user", "content": "a"}, {"role": "user", "content": "b"}]
    out = render(tpl, bad, bos="[BOS]")
    assert not out.get("ok") and "Conversation roles must alternate" in out["error"]
    good = render(tpl, [{"role": "user", "content": "a"}, {"role": "assistant", "content": "b"}], bos="[BOS]")
    assert good["text"] == "[BOS]ab"


def test_loop_controls_and_reverse_slices():
    tpl = "{% for m in messages %}{% if m['role'] == 'system' %}{% continue %}{% endif %}{{ m['content'] }}|{% endfor %}"
    assert render(tpl, SYSTEM + CHAT)["text"] == "".join(m["content"] + "|" for m in CHAT)
    tpl = "{% for m in messages %}{% if loop.index0 == 1 %}{% break %}{% endif %}{{ m['content'] }}{% endfor %}"
    assert render(tpl, CHAT)["text"] == CHAT[0]["content"]
    tpl = "{% for m in messages[::-1] %}{{ m['role'][0] }}{% endfor %}"      # python slice idiom of some templates
    assert render(tpl, CHAT)["text"] == "uau"


def test_strftime_now_and_generation_markers():
    tpl = "{% generation %}{{ strftime_now('%Y') }}{% endgeneration %}{% if add_generation_prompt %}>{% endif %}"
    assert render(tpl, CHAT, True)["text"] == str(datetime.datetime.now().year) + ">"
    assert render(tpl, CHAT, False)["text"] == str(datetime.datetime.now().year)


def test_list_content_is_flattened_with_image_placeholders():
    msgs = [{"role": "user", "content": [{"type": "text", "text": "What is this?"},
                                         {"type": "image_url", "image_url": {"url": "http://x/y.png"}}]}]
    tpl = "{% for m in messages %}{{ m['content'] }}{% endfor %}"
    assert render(tpl, msgs)["text"] == "What is this?![](http://x/y.png)"


def test_tools_go_to_templates_that_know_them_and_into_the_last_turn_otherwise():
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]
    aware = "{% if tools %}T:{{ tools | length }};{% endif %}{% for m in messages %}{{ m['content'] }}{% endfor %}"
    assert render(aware, CHAT[:1], tools=tools, tool_prompt="Use: ")["text"] == "T:1;Hello, how are you?\n---\nUse: "
    plain = "{% for m in messages %}{{ m['content'] }}{% endfor %}"
    text = render(plain, CHAT[:1], tools=tools, tool_prompt="Use them.")["text"]
    assert text.startswith('Hello, how are you?\n---\n[{"type":"function"') and text.endswith("]\nUse them.")


def test_a_trailing_assistant_message_is_continued():
    """The rendered prompt ends right after the assistant's partial answer: no end-of-turn marker, no new
    generation prompt (the reference's continue_final_message behaviour)."""
    tpl = ("{% for m in messages %}<|{{ m['role'] }}|>{{ m['content'] }}</s>\n{% endfor %}"
           "{% if add_generation_prompt %}<|assistant|>{% endif %}")
    msgs = [{"role": "user", "content": "Which is bigger?"}, {"role": "assistant", "content": "the elephant, but "}]
    assert render(tpl, msgs, True)["text"] == "<|user|>Which is bigger?</s>\n<|assistant|>the elephant, but"
    # a conversation that ends with the user is rendered as before
    assert render(tpl, msgs[:1], True)["text"] == "<|user|>Which is bigger?</s>\n<|assistant|>"


def test_missing_template_is_an_error():
    pybridge._STATE.update(chat_template=None)
    out = json.loads(pybridge.apply_chat_template(json.dumps(dict(messages=CHAT))))
    assert not out.get("ok") and "no chat template" in out["error"]


def test_template_files_beside_the_tokenizer_config(tmp_path):
    """chat_template.json overrides tokenizer_config.json; processor_config.json and chat_template.jinja are read when
    nothing else defines a template."""
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"chat_template": "from-tokenizer-config"}))
    out = json.loads(pybridge.load(json.dumps({"tokenizer_name": str(tmp_path)})))
    assert out["has_chat_template"] and pybridge._STATE["chat_template"] == "from-tokenizer-config"
    (tmp_path / "processor_config.json").write_text(json.dumps({"chat_template": "from-processor", "image_seq_len": 169}))
    pybridge.load(json.dumps({"tokenizer_name": str(tmp_path)}))
    assert pybridge._STATE["chat_template"] == "from-processor"
    (tmp_path / "chat_template.json").write_text(json.dumps({"chat_template": "stand-alone"}))
    pybridge.load(json.dumps({"tokenizer_name": str(tmp_path)}))
    assert pybridge._STATE["chat_template"] == "stand-alone"
    other = tmp_path / "jinja"
    other.mkdir()
    (other / "chat_template.jinja").write_text("{{ messages[0]['content'] }}!")
    pybridge.load(json.dumps({"tokenizer_name": str(other)}))
    assert json.loads(pybridge.apply_chat_template(json.dumps(dict(messages=CHAT))))["text"] == CHAT[0]["content"] + "!"
