"""Operator schema parser and dispatch registry.

Reference: ft-dispatch/src/lib.rs - ``parse_schema_name`` :1153 (namespace stripping, overload
validation, trailing-underscore in-place marker), ``parse_schema_or_name`` :1216,
``SchemaRegistry.register/lookup`` :1040/:1101 (duplicate detection, keyset validation,
unsupported base operators), ``digest64`` :1144 (FNV-1a).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple, Union

from ..runtime import native
from .keys import DispatchKeyError, DispatchKeySet

DISPATCHABLE_BASES = ("add", "sub", "mul", "div", "matmul", "dot", "outer", "bmm", "min", "max",
                      "atan2", "fmod", "remainder")


class OpSchemaError(ValueError):
    pass


class SchemaRegistryError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


def digest64(text: str) -> int:
    return native.fnv1a64(text.encode("utf-8"))


_IDENT = re.compile(r"^[A-Za-z_][A-Za-z0-9_]*$")


@dataclass(frozen=True)
class OpSchemaName:
    base: str
    overload: Optional[str]
    is_inplace: bool

    def unambiguous_name(self) -> str:
        name = self.base + ("_" if self.is_inplace else "")
        return f"{name}.{self.overload}" if self.overload else name


@dataclass(frozen=True)
class SchemaArgument:
    type: str
    name: str
    default: Optional[str]
    kwarg_only: bool
    alias: Optional[str]


@dataclass(frozen=True)
class ParsedOpSchema:
    op: OpSchemaName
    arguments: Tuple[SchemaArgument, ...]
    returns: str
    is_out_variant: bool
    schema_digest: int


def parse_schema_name(text: str) -> OpSchemaName:
    t = text.strip()
    if not t:
        raise OpSchemaError("empty schema input")
    op = t.rsplit("::", 1)[1] if "::" in t else t
    if not op:
        raise OpSchemaError("invalid operator name: missing operator token after namespace")
    overload = None
    if "." in op:
        raw_base, overload = op.split(".", 1)
        if not overload or overload == "default" or overload.startswith("__") or not _IDENT.match(overload):
            raise OpSchemaError(f"invalid overload name '{overload}'")
    else:
        raw_base = op
    if not raw_base:
        raise OpSchemaError("invalid operator name: empty base operator name")
    is_inplace = raw_base.endswith("_")
    base = raw_base.rstrip("_") if is_inplace else raw_base
    if not base or not _IDENT.match(base):
        raise OpSchemaError("invalid operator name: operator base contains invalid characters")
    return OpSchemaName(base, overload, is_inplace)


def _split_top_level(s: str) -> List[str]:
    parts, depth, cur = [], 0, []
    for ch in s:
        if ch in "([":
            depth += 1
        elif ch in ")]":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append("".join(cur).strip())
            cur = []
        else:
            cur.append(ch)
    if "".join(cur).strip():
        parts.append("".join(cur).strip())
    return parts


def parse_schema_or_name(text: str) -> Union[OpSchemaName, ParsedOpSchema]:
    t = text.strip()
    if not t:
        raise OpSchemaError("empty schema input")
    if "(" not in t:
        if "->" in t or ")" in t:
            raise OpSchemaError("malformed schema: unbalanced parentheses")
        return parse_schema_name(t)
    head, rest = t.split("(", 1)
    name = parse_schema_name(head)
    # find the matching close parenthesis of the argument list
    depth, close = 1, -1
    for i, ch in enumerate(rest):
        if ch == "(":
            depth += 1
        elif ch == ")":
            depth -= 1
            if depth == 0:
                close = i
                break
    if close < 0:
        raise OpSchemaError("malformed schema: missing ')' after the argument list")
    args_text, tail = rest[:close], rest[close + 1:].strip()
    if not tail.startswith("->"):
        raise OpSchemaError("malformed schema: missing '->' return annotation")
    returns = tail[2:].strip()
    if not returns:
        raise OpSchemaError("malformed schema: empty return type")
    args: List[SchemaArgument] = []
    kw_only = False
    for part in _split_top_level(args_text):
        if part == "*":
            kw_only = True
            continue
        default = None
        if "=" in part:
            part, default = (x.strip() for x in part.split("=", 1))
        toks = part.rsplit(" ", 1)
        if len(toks) != 2 or not _IDENT.match(toks[1]):
            raise OpSchemaError(f"malformed schema argument '{part}'")
        ty, an = toks[0].strip(), toks[1]
        alias = None
        m = re.search(r"\(([a-z])(!?)\)", ty)
        if m:
            alias = m.group(1) + m.group(2)
        args.append(SchemaArgument(ty, an, default, kw_only, alias))
    is_out = name.overload == "out" or any(a.kwarg_only and a.alias and a.alias.endswith("!") for a in args)
    normalized = f"{name.unambiguous_name()}({args_text.strip()}) -> {returns}"
    return ParsedOpSchema(name, tuple(args), returns, is_out, digest64(normalized))


@dataclass(frozen=True)
class SchemaDispatchEntry:
    normalized_name: str
    op: str
    keyset: DispatchKeySet
    is_out_variant: bool
    schema_digest: int


class SchemaRegistry:
    def __init__(self):
        self._entries: Dict[str, SchemaDispatchEntry] = {}

    def __len__(self):
        return len(self._entries)

    def register(self, parsed: Union[OpSchemaName, ParsedOpSchema], keyset: DispatchKeySet) -> str:
        try:
            keyset.validate_for_scalar_binary()
        except DispatchKeyError as e:
            raise SchemaRegistryError("IncompatibleDispatchKeyset", f"schema dispatch keyset is incompatible: {e}")
        if isinstance(parsed, ParsedOpSchema):
            name, is_out, digest = parsed.op, parsed.is_out_variant, parsed.schema_digest
        else:
            name, is_out, digest = parsed, False, digest64(parsed.unambiguous_name())
        normalized = name.unambiguous_name()
        if normalized in self._entries:
            raise SchemaRegistryError("DuplicateSchema", f"schema registry already has an entry for '{normalized}'")
        if name.base not in DISPATCHABLE_BASES:
            raise SchemaRegistryError("UnsupportedOperator", f"schema base operator '{name.base}' is not yet dispatchable")
        self._entries[normalized] = SchemaDispatchEntry(normalized, name.base, keyset, is_out, digest)
        return normalized

    def lookup(self, normalized_name: str) -> SchemaDispatchEntry:
        e = self._entries.get(normalized_name)
        if e is None:
            raise SchemaRegistryError("MissingSchema", f"schema registry has no entry for '{normalized_name}'")
        return e

    def __iter__(self):
        return iter(sorted(self._entries.values(), key=lambda e: e.normalized_name))
