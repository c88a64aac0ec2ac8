from allie_b200.evaluation.chess_llm import ChessLLM, openai_completion  # noqa: F401
