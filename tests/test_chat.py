"""Chat templates against the reference's own known-answer test (crates/ksearch_gguf/src/tokenizer.rs:147-163)."""
from ksearch_b200.chat import gemma4_chat_from_messages, gemma4_chat_prompt
from ksearch_b200.scheduler import BUILTIN_STOPS


def test_reference_known_answer():
    prompt = gemma4_chat_from_messages([("system", "be brief"), ("user", "Hi"), ("assistant", "Hi!"), ("user", "again")])
    assert prompt == ("<|turn>system\n<|think|>\nbe brief<turn|>\n<|turn>user\nHi<turn|>\n<|turn>model\nHi!<turn|>\n"
                      "<|turn>user\nagain<turn|>\n<|turn>model\n")
    assert gemma4_chat_prompt("Hi") == "<|turn>user\nHi<turn|>\n<|turn>model\n"


def test_roles_and_system_turns():
    assert gemma4_chat_from_messages([]) == "<|turn>model\n"
    assert gemma4_chat_from_messages([("user", "a")]) == gemma4_chat_prompt("a")
    two = gemma4_chat_from_messages([("system", "x"), ("user", "q"), ("system", "y")])
    assert two.startswith("<|turn>system\n<|think|>\nx\n\ny<turn|>\n") and two.endswith("<|turn>user\nq<turn|>\n<|turn>model\n")
    assert "<|turn>user\nt<turn|>" in gemma4_chat_from_messages([("tool", "t")])     # unknown roles speak as the user
    assert all(s in BUILTIN_STOPS for s in ("<turn|>", "<|turn>"))                  # the markers the scheduler stops on
