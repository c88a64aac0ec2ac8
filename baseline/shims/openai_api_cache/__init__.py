"""Import stand-in for ``openai-api-cache`` (a Redis-backed cache in front of the OpenAI client, not
installed and not reachable here).  Constructing it fails with a clear message."""


class OpenAIAPICache:
    def __init__(self, *args, **kwargs):
        raise NotImplementedError("openai-api-cache needs a Redis server and network access")
