"""The OpenAI Python client against a local ``orinfer serve`` (pip install openai).

    python examples/openai-python.py http://127.0.0.1:8080/v1
"""
import json
import sys

from openai import OpenAI

client = OpenAI(base_url=sys.argv[1] if len(sys.argv) > 1 else "http://127.0.0.1:8080/v1",
                api_key="unused")

# streaming chat
for chunk in client.chat.completions.create(
        model="default", stream=True, max_tokens=64,
        messages=[{"role": "user", "content": "Name three rivers."}]):
    if chunk.choices and chunk.choices[0].delta.content:
        print(chunk.choices[0].delta.content, end="", flush=True)
print()

# output constrained to a JSON schema
schema = {"type": "object", "properties": {"river": {"type": "string"},
                                            "length_km": {"type": "integer"}},
          "required": ["river", "length_km"], "additionalProperties": False}
reply = client.chat.completions.create(
    model="default", max_tokens=64,
    messages=[{"role": "user", "content": "The longest river in Europe, as JSON."}],
    response_format={"type": "json_schema", "json_schema": {"name": "river", "schema": schema}})
print(json.loads(reply.choices[0].message.content))

# embeddings (served by encoder models and, mean-pooled, by decoders)
vectors = client.embeddings.create(model="default", input=["a river", "a mountain"])
print(len(vectors.data), "vectors of", len(vectors.data[0].embedding), "dimensions")
