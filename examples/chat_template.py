"""Chat templates: detection by model name and formatting of a conversation."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
from realizar_b200.serving.chat_template import ChatMessage, auto_detect_template, create_template

msgs = [ChatMessage.system("You are terse."), ChatMessage.user("Hi"), ChatMessage.assistant("Hello."), ChatMessage.user("Bye")]
for name in ("qwen2.5-7b-instruct", "llama-2-7b-chat", "mistral-7b-instruct", "phi-2", "zephyr-7b"):
    t = auto_detect_template(name)
    print(f"--- {name}: {t.format}\n{t.format_conversation(msgs)}")
print(create_template("alpaca").format_conversation(msgs))
