from allie_b200.evaluation.annotate import annotate, annotate_row, main  # noqa: F401

if __name__ == "__main__":
    main()
