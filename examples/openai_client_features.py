"""Requests against a running server (`python -m vllm_torchtpu_b200 serve <model> --port 8000`): sampling
parameters, stop strings, several completions per prompt, function calling, tokenize.  Standard library only.
`python examples/openai_client_features.py --url http://127.0.0.1:8000`"""
import argparse
import json
import urllib.request


def post(url: str, path: str, body: dict) -> dict:
    req = urllib.request.Request(url + path, method="POST", headers={"Content-Type": "application/json"},
                                 data=json.dumps(body).encode())
    with urllib.request.urlopen(req, timeout=300) as r:
        return json.loads(r.read())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    a = ap.parse_args(argv)
    r = post(a.url, "/v1/completions", {
        "prompt": "Three facts about tensor memory:", "max_tokens": 64, "temperature": 0.8, "top_p": 0.95, "min_p": 0.05,
        "frequency_penalty": 0.3, "presence_penalty": 0.2, "n": 2, "stop": ["\n\n"]})
    for ch in r["choices"]:
        print(f"[{ch['index']}] {ch['finish_reason']}: {ch['text']!r}")
    tools = [{"type": "function", "function": {"name": "get_weather", "description": "current weather of a city",
                                               "parameters": {"type": "object", "properties": {
                                                   "city": {"type": "string"}, "unit": {"enum": ["C", "F"]}},
                                                   "required": ["city", "unit"]}}}]
    r = post(a.url, "/v1/chat/completions", {
        "messages": [{"role": "user", "content": "What is the weather in Paris?"}], "tools": tools, "max_tokens": 64,
        "tool_choice": {"type": "function", "function": {"name": "get_weather"}}, "temperature": 0})
    msg = r["choices"][0]["message"]
    print("tool calls:", [(c["function"]["name"], c["function"]["arguments"]) for c in msg.get("tool_calls", [])])
    print("tokens:", post(a.url, "/tokenize", {"prompt": "tensor memory"})["count"])


if __name__ == "__main__":
    main()
