"""The one exception raised for a kernel function that cannot be compiled or run as asked.

Same convention as the reference's KernelError (src/autokernel/errors.py:11-24): when the complaint is about a
line of the user's code the message starts with `file:line:` and quotes the line, and it is raised before
anything runs.
"""

from __future__ import annotations

import ast
import linecache


class KernelError(Exception):
    def __init__(self, message: str, *, filename: str | None = None, node: ast.AST | None = None) -> None:
        lineno = getattr(node, "lineno", None)
        if filename and lineno:
            message = f"{filename}:{lineno}: {message}"
            line = linecache.getline(filename, lineno).strip()
            if line:
                message += f"\n    {line}"
        super().__init__(message)
