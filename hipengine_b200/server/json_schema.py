"""Stdlib-only JSON Schema subset validator used for ``response_format`` and tool parameters.

Supported keywords (the subset the reference documents, ``hipengine/server/json_schema.py``; ``docs/API.md``
structured-output section): type, enum, const, properties, required, additionalProperties, items,
prefixItems, min/max (Length, Items, Properties, imum, exclusive*), multipleOf, pattern, allOf / anyOf / oneOf /
not, if / then / else and local ``$ref`` (``#/...``).  Unknown keywords are ignored, as JSON Schema prescribes.
"""
from __future__ import annotations

import re
from typing import Any, List, Optional

_TYPES = {
    "object": lambda v: isinstance(v, dict),
    "array": lambda v: isinstance(v, list),
    "string": lambda v: isinstance(v, str),
    "boolean": lambda v: isinstance(v, bool),
    "null": lambda v: v is None,
    "integer": lambda v: (isinstance(v, int) and not isinstance(v, bool)) or (isinstance(v, float) and v.is_integer()),
    "number": lambda v: isinstance(v, (int, float)) and not isinstance(v, bool),
}


class SchemaError(ValueError):
    """The schema itself is malformed or uses an unresolvable reference."""


def _resolve(root: Any, ref: str) -> Any:
    if not ref.startswith("#"):
        raise SchemaError(f"only local $ref is supported, got {ref!r}")
    node = root
    for part in ref[1:].split("/"):
        if not part:
            continue
        part = part.replace("~1", "/").replace("~0", "~")
        if isinstance(node, dict) and part in node:
            node = node[part]
        elif isinstance(node, list) and part.isdigit() and int(part) < len(node):
            node = node[int(part)]
        else:
            raise SchemaError(f"unresolvable $ref {ref!r}")
    return node


def validate(instance: Any, schema: Any, root: Optional[Any] = None, path: str = "$", depth: int = 0) -> List[str]:
    """Returns a list of violation messages (empty = valid)."""
    if root is None:
        root = schema
    if depth > 64:
        return [f"{path}: schema recursion too deep"]
    if schema is True or schema == {}:
        return []
    if schema is False:
        return [f"{path}: schema forbids any value"]
    if not isinstance(schema, dict):
        raise SchemaError(f"schema at {path} must be an object or boolean")
    errs: List[str] = []
    if "$ref" in schema:
        errs += validate(instance, _resolve(root, schema["$ref"]), root, path, depth + 1)
    t = schema.get("type")
    if t is not None:
        types = t if isinstance(t, list) else [t]
        if not any(_TYPES.get(x, lambda v: False)(instance) for x in types):
            return errs + [f"{path}: expected type {t}, got {type(instance).__name__}"]
    if "enum" in schema and instance not in schema["enum"]:
        errs.append(f"{path}: value not in enum")
    if "const" in schema and instance != schema["const"]:
        errs.append(f"{path}: value differs from const")
    if isinstance(instance, (int, float)) and not isinstance(instance, bool):
        if "minimum" in schema and instance < schema["minimum"]:
            errs.append(f"{path}: below minimum {schema['minimum']}")
        if "maximum" in schema and instance > schema["maximum"]:
            errs.append(f"{path}: above maximum {schema['maximum']}")
        if "exclusiveMinimum" in schema and instance <= schema["exclusiveMinimum"]:
            errs.append(f"{path}: not above exclusiveMinimum")
        if "exclusiveMaximum" in schema and instance >= schema["exclusiveMaximum"]:
            errs.append(f"{path}: not below exclusiveMaximum")
        if "multipleOf" in schema and schema["multipleOf"]:
            q = instance / schema["multipleOf"]
            if abs(q - round(q)) > 1e-9:
                errs.append(f"{path}: not a multiple of {schema['multipleOf']}")
    if isinstance(instance, str):
        if "minLength" in schema and len(instance) < schema["minLength"]:
            errs.append(f"{path}: shorter than minLength")
        if "maxLength" in schema and len(instance) > schema["maxLength"]:
            errs.append(f"{path}: longer than maxLength")
        if "pattern" in schema:
            try:
                if re.search(schema["pattern"], instance) is None:
                    errs.append(f"{path}: does not match pattern")
            except re.error as exc:
                raise SchemaError(f"bad pattern at {path}: {exc}") from None
    if isinstance(instance, list):
        if "minItems" in schema and len(instance) < schema["minItems"]:
            errs.append(f"{path}: fewer than minItems")
        if "maxItems" in schema and len(instance) > schema["maxItems"]:
            errs.append(f"{path}: more than maxItems")
        prefix = schema.get("prefixItems", [])
        for i, sub in enumerate(prefix[:len(instance)]):
            errs += validate(instance[i], sub, root, f"{path}[{i}]", depth + 1)
        if "items" in schema:
            for i in range(len(prefix), len(instance)):
                errs += validate(instance[i], schema["items"], root, f"{path}[{i}]", depth + 1)
        if schema.get("uniqueItems") and len({repr(x) for x in instance}) != len(instance):
            errs.append(f"{path}: items are not unique")
    if isinstance(instance, dict):
        props = schema.get("properties", {})
        for k in schema.get("required", []):
            if k not in instance:
                errs.append(f"{path}: missing required property {k!r}")
        for k, sub in props.items():
            if k in instance:
                errs += validate(instance[k], sub, root, f"{path}.{k}", depth + 1)
        ap = schema.get("additionalProperties", True)
        extra = [k for k in instance if k not in props]
        if ap is False and extra:
            errs.append(f"{path}: additional properties not allowed: {extra[:4]}")
        elif isinstance(ap, dict):
            for k in extra:
                errs += validate(instance[k], ap, root, f"{path}.{k}", depth + 1)
        if "minProperties" in schema and len(instance) < schema["minProperties"]:
            errs.append(f"{path}: fewer than minProperties")
        if "maxProperties" in schema and len(instance) > schema["maxProperties"]:
            errs.append(f"{path}: more than maxProperties")
    for sub in schema.get("allOf", []):
        errs += validate(instance, sub, root, path, depth + 1)
    if "anyOf" in schema and not any(not validate(instance, s, root, path, depth + 1) for s in schema["anyOf"]):
        errs.append(f"{path}: matches none of anyOf")
    if "oneOf" in schema:
        n = sum(1 for s in schema["oneOf"] if not validate(instance, s, root, path, depth + 1))
        if n != 1:
            errs.append(f"{path}: matches {n} of oneOf (need exactly 1)")
    if "not" in schema and not validate(instance, schema["not"], root, path, depth + 1):
        errs.append(f"{path}: matches the schema under not")
    if "if" in schema:
        branch = "then" if not validate(instance, schema["if"], root, path, depth + 1) else "else"
        if branch in schema:
            errs += validate(instance, schema[branch], root, path, depth + 1)
    return errs


# keywords that constrain instances and that ``validate`` does not implement: ignoring them would accept outputs the
# caller's schema forbids, so a schema using them is refused
UNSUPPORTED_KEYWORDS = ("patternProperties", "propertyNames", "dependentRequired", "dependentSchemas", "dependencies",
                        "contains", "minContains", "maxContains", "unevaluatedProperties", "unevaluatedItems",
                        "$dynamicRef", "$recursiveRef", "contentEncoding", "contentMediaType", "contentSchema")
_SCHEMA_MAPS = ("properties", "$defs", "definitions")
_SCHEMA_SINGLE = ("items", "additionalProperties", "not", "if", "then", "else")
_SCHEMA_LISTS = ("allOf", "anyOf", "oneOf", "prefixItems")


def check_schema(schema: Any) -> None:
    """Reject schemas this validator cannot honour (raises ``SchemaError``): a non-local ``$ref`` or one that does not
    resolve, a pattern that does not compile, an unknown type name, a constraining keyword outside the subset.  The
    walk follows the positions where JSON Schema puts subschemas, so a *property* that happens to be called
    ``contains`` or ``type`` is not mistaken for a keyword."""
    def walk(node: Any, where: str) -> None:
        if isinstance(node, bool):
            return
        if not isinstance(node, dict):
            raise SchemaError(f"{where}: a schema must be an object or a boolean")
        for k in UNSUPPORTED_KEYWORDS:
            if k in node:
                raise SchemaError(f"{where}: keyword {k!r} is not supported")
        if "$ref" in node:
            _resolve(schema, node["$ref"])
        if "pattern" in node:
            try:
                re.compile(node["pattern"])
            except (re.error, TypeError) as exc:
                raise SchemaError(f"{where}: bad pattern: {exc}") from None
        if "type" in node:
            types = node["type"] if isinstance(node["type"], list) else [node["type"]]
            for t in types:
                if t not in _TYPES:
                    raise SchemaError(f"{where}: unknown type {t!r}")
        for k in _SCHEMA_MAPS:
            if isinstance(node.get(k), dict):
                for name, sub in node[k].items():
                    walk(sub, f"{where}/{k}/{name}")
        for k in _SCHEMA_SINGLE:
            if k in node:
                walk(node[k], f"{where}/{k}")
        for k in _SCHEMA_LISTS:
            if isinstance(node.get(k), list):
                for n, sub in enumerate(node[k]):
                    walk(sub, f"{where}/{k}/{n}")
    if not isinstance(schema, (dict, bool)):
        raise SchemaError("schema must be an object or boolean")
    walk(schema, "#")
