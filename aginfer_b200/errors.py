"""User-facing failure types of the packaging tool.

Same three classes (and names) as the reference's ``src/aginfer/errors.py:1-14`` so
that callers' ``except`` clauses and tests carry over unchanged.
"""


class AgInferError(Exception):
    """Root of every deterministic packaging failure."""


class ValidationError(AgInferError):
    """An input (checkpoint, plan, artifact, target) is malformed or unsupported."""


class FormatError(AgInferError):
    """An AIM container or binary plan failed a structural or integrity check."""


class CompatibilityError(AgInferError):
    """The package holds no variant for the requested target."""
