from nanotitan_b200.data.prepare_dataset import main  # noqa: F401

if __name__ == "__main__":
    main()
