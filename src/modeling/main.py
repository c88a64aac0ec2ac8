from allie_b200.train.main import main

if __name__ == "__main__":
    main()
