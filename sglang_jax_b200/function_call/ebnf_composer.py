"""Builds an EBNF grammar that forces well-formed tool calls for `tool_choice="required"` or a
named function (reference `python/sgl_jax/srt/function_call/ebnf_composer.py`)."""

from __future__ import annotations

import json

_JSON_RULES = r'''
json_value ::= json_object | json_array | json_string | json_number | "true" | "false" | "null"
json_object ::= "{" ws ( json_member ( ws "," ws json_member )* )? ws "}"
json_member ::= json_string ws ":" ws json_value
json_array ::= "[" ws ( json_value ( ws "," ws json_value )* )? ws "]"
json_string ::= "\"" ( [^"\\] | "\\" . )* "\""
json_number ::= "-"? [0-9]+ ( "." [0-9]+ )? ( [eE] [+-]? [0-9]+ )?
ws ::= [ \n\t]*
'''


class EBNFComposer:
    @staticmethod
    def _fn(tool):
        fn = tool.function if hasattr(tool, "function") else tool["function"]
        name = fn.name if hasattr(fn, "name") else fn["name"]
        params = fn.parameters if hasattr(fn, "parameters") else fn.get("parameters")
        return name, params or {}

    @classmethod
    def build_ebnf(cls, tools, call_template: str = '{{"name": "{name}", "arguments": {args}}}',
                   begin: str = "<tool_call>\n", end: str = "\n</tool_call>", separator: str = "\n",
                   function_name: str | None = None) -> str:
        rules, alts = [], []
        for i, t in enumerate(tools):
            name, params = cls._fn(t)
            if function_name and name != function_name:
                continue
            props = params.get("properties", {})
            required = params.get("required", [])
            members = []
            for k in props:
                members.append(f'"\\"{k}\\"" ws ":" ws json_value')
            if members:
                req = [m for k, m in zip(props, members) if k in required] or members[:1]
                body = ' ws "," ws '.join(req)
                args_rule = f'"{{" ws {body} ( ws "," ws json_member )* ws "}}"'
            else:
                args_rule = "json_object"
            rules.append(f"args_{i} ::= {args_rule}")
            lit = call_template.format(name=name, args="\x00").split("\x00")
            alts.append(f'call_{i}')
            rules.append(f"call_{i} ::= {json.dumps(lit[0])} args_{i} {json.dumps(lit[1])}")
        root = f'root ::= {json.dumps(begin)} ( {" | ".join(alts)} ) {json.dumps(end)} ' \
               f'( {json.dumps(separator + begin)} ( {" | ".join(alts)} ) {json.dumps(end)} )*'
        return root + "\n" + "\n".join(rules) + _JSON_RULES
