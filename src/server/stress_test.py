from allie_b200.serve.stress_test import main, query, run  # noqa: F401

if __name__ == "__main__":
    main()
