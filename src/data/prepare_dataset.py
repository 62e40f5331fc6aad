from nanotitan_b200.data.prepare_dataset import main, tokenize_split, write_token_file  # noqa: F401

if __name__ == "__main__":
    main()
