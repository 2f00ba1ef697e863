"""Chat front end: prompt rendering, reasoning split, tool-call parsing, response assembly.

Fills the role of the reference's ``crates/blaze-chat`` crate (``render`` / ``parser`` / ``think`` / ``tool_call`` /
``openai`` modules, itself vendored from SGLang's processor).
"""
from .template import ChatFormatter  # noqa: F401
from .reasoning import ThinkParser, get_think_parser  # noqa: F401
from .tools import ToolCall, ToolParser, get_tool_parser  # noqa: F401
from .processor import ChatResponseProcessor  # noqa: F401
