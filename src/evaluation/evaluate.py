from allie_b200.evaluation.evaluate import evaluate, evaluate_quick, evaluate_value, main  # noqa: F401

if __name__ == "__main__":
    main()
