from allie_b200.serve.server import main

if __name__ == "__main__":
    main()
